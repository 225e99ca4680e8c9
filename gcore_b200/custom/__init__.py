from .registry import load_custom_module, load_custom_module_registry, register_custom_module  # noqa: F401
