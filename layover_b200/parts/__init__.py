from .base import (
    PagedKVNeed, Part, PartSpec, Runtime, StateNeed, build_part, register_block, register_feed_forward,
    register_mixer, register_norm, register_position, registered, unregister, walk_parts,
)
from . import norm, position, feed_forward, attention, block  # noqa: F401  (fill the registries)
from .attention import Attention, attention_spec
from .block import PreNormBlock
from .feed_forward import GatedMLP
from .norm import RMSNorm
from .position import RotaryHalf

__all__ = [
    "PagedKVNeed", "Part", "PartSpec", "Runtime", "StateNeed", "build_part", "register_block",
    "register_feed_forward", "register_mixer", "register_norm", "register_position", "registered", "unregister",
    "walk_parts",
    "Attention", "attention_spec", "PreNormBlock", "GatedMLP", "RMSNorm", "RotaryHalf",
]
