from .qwen2 import ConfigError, Qwen2Config
from .registry import (
    architecture_of,
    known_architectures,
    read_config,
    register_architecture,
    resolve,
    unregister_architecture,
)
