from .base import (
    DTYPE_BYTES,
    Architecture,
    load_config,
    read_config_json,
    register_architecture,
    resolve_architecture,
    supported_architectures,
    unregister_architecture,
)
from .qwen3 import PRESETS, Qwen3Config, preset

__all__ = [
    "DTYPE_BYTES", "Architecture", "load_config", "read_config_json", "register_architecture",
    "resolve_architecture", "supported_architectures", "unregister_architecture",
    "PRESETS", "Qwen3Config", "preset",
]
