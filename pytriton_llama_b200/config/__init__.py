from .llama import ConfigError, LlamaConfig, RopeScaling  # noqa: F401
from .engine import EngineConfig  # noqa: F401
from .registry import (known_architectures, read_config_json, register_architecture,  # noqa: F401
                       resolve_architecture)
