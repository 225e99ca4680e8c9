from .config_checks import check_rollout_batches, find_risky_settings, run_config_checks  # noqa: F401
