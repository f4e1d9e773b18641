"""Configuration: typed readers of config.json and the architecture registry."""
from .reader import ConfigError, KeyReader, read_config_json
from .registry import (Architecture, register_architecture, unregister_architecture,
                       registered_architectures, lookup_architecture, architecture_name,
                       parse_config, load_config)
from .qwen2_moe import Qwen2MoeConfig

__all__ = ["ConfigError", "KeyReader", "read_config_json", "Architecture", "register_architecture",
           "unregister_architecture", "registered_architectures", "lookup_architecture",
           "architecture_name", "parse_config", "load_config", "Qwen2MoeConfig"]
