from .runner import EvaluateRunner, pass_at_k  # noqa: F401
