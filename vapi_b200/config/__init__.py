"""The architecture registry (config.json -> model) and run-time configuration (TOML / flags)."""
from .model import (Architecture, ConfigError, eos_token_ids, load_config_json, register_architecture,
                    registered_architectures, resolve_architecture, unregister_architecture)

__all__ = ["Architecture", "ConfigError", "eos_token_ids", "load_config_json",
           "register_architecture", "registered_architectures", "resolve_architecture",
           "unregister_architecture"]
