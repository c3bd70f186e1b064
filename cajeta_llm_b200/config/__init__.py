from .base import (Architecture, ConfigError, ConfigReader, ModelConfig, get_architecture, load_config,  # noqa: F401
                   parse_config_dict, register_architecture, registered_architectures, unregister_architecture)
