"""``training_engine_tensor.engine_config``: the run-time configuration under the reference's module
name (its engine_config.py:132-441). Everything lives in :mod:`forgetrain_b200.engine_config`."""
from forgetrain_b200.engine_config import (  # noqa: F401
    DECLARED_ENV_VARS, EXTERNAL_ENV_WHITELIST, LEGACY_FIELD_ALIASES, LEGACY_NOOP_FIELDS, EngineConfig,
    env_table_markdown, from_env, from_legacy, from_spec, get_config, has_global_config,
    print_config_summary, register_reset_hook, reset_global_config, set_global_config, validate_config)

__all__ = ["EngineConfig", "from_env", "from_legacy", "from_spec", "set_global_config", "get_config",
           "has_global_config", "register_reset_hook", "reset_global_config", "print_config_summary",
           "validate_config", "DECLARED_ENV_VARS", "EXTERNAL_ENV_WHITELIST"]
