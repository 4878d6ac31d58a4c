from .model_config import LlamaConfig, RopeScaling, read_config_json, write_config_json
from .engine_config import EngineConfig, parse_dtype
from .registry import (Architecture, register_architecture, unregister_architecture,
                       known_architectures, architecture_for)

__all__ = ["LlamaConfig", "RopeScaling", "read_config_json", "write_config_json", "EngineConfig",
           "parse_dtype", "Architecture", "register_architecture", "unregister_architecture",
           "known_architectures", "architecture_for"]
