from .model_config import ConfigError, Qwen2MoeConfig, load_config_json  # noqa: F401
from .registry import (config_from_dir, config_from_json, known_architectures,  # noqa: F401
                       lookup, register_architecture)
