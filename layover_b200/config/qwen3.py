"""Typed configuration of Qwen3 dense, read from its own config.json keys.

Keys, defaults and refusals follow layover/config.py:28-59 of the reference: `head_dim` is read
and not derived (Qwen3-4B stores 128 while hidden/heads is 80), `num_key_value_heads` defaults
to the number of heads, `rope_theta` may sit at the top level or inside `rope_parameters` /
`rope_scaling`, sliding windows and non-default rope types are refused.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

from .base import DTYPE_BYTES


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    eos_token_id: int | None = None
    bos_token_id: int | None = None

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    def __post_init__(self):
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ValueError(f"{name} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2:
            raise ValueError(f"head_dim must be even for rotary embeddings, got {self.head_dim}")
        if not self.rms_norm_eps > 0 or not self.rope_theta > 0:
            raise ValueError("rms_norm_eps and rope_theta must be positive")

    @classmethod
    def from_hf_dict(cls, raw: dict) -> "Qwen3Config":
        if raw.get("model_type", cls.model_type) != cls.model_type:
            raise ValueError(f"unsupported model_type {raw['model_type']!r}")
        if raw.get("use_sliding_window"):
            raise ValueError("sliding-window attention is not supported")
        rope = raw.get("rope_parameters") or raw.get("rope_scaling") or {}
        if rope.get("rope_type", rope.get("type", "default")) != "default":
            raise ValueError(f"unsupported rope configuration {rope!r}")
        for key in ("attention_bias", "mlp_bias"):
            if raw.get(key):
                raise ValueError(f"{key} is not supported: the reference's layers have no bias")
        if raw.get("hidden_act", "silu") != "silu":
            raise ValueError(f"unsupported hidden_act {raw['hidden_act']!r}")
        missing = [k for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                               "num_attention_heads", "max_position_embeddings") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks {missing}")
        eos = raw.get("eos_token_id")
        return cls(
            vocab_size=raw["vocab_size"],
            hidden_size=raw["hidden_size"],
            intermediate_size=raw["intermediate_size"],
            num_hidden_layers=raw["num_hidden_layers"],
            num_attention_heads=raw["num_attention_heads"],
            num_key_value_heads=raw.get("num_key_value_heads") or raw["num_attention_heads"],
            head_dim=raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"],
            max_position_embeddings=raw["max_position_embeddings"],
            rope_theta=float(raw.get("rope_theta", rope.get("rope_theta", 10000.0))),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", True)),
            eos_token_id=eos[0] if isinstance(eos, list) else eos,
            bos_token_id=raw.get("bos_token_id"),
        )

    def to_hf_dict(self) -> dict:
        """The config.json that reads back as this configuration (layover/config.py:104-126)."""
        return {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "attention_dropout": 0.0,
            "use_sliding_window": False,
            "sliding_window": None,
            "max_window_layers": self.num_hidden_layers,
            "eos_token_id": self.eos_token_id,
            "bos_token_id": self.bos_token_id,
        }

    def replace(self, **changes) -> "Qwen3Config":
        return replace(self, **changes)

    @property
    def kv_groups(self) -> int:
        """Query heads that read each KV head (layover/config.py:91-96)."""
        return self.num_attention_heads // self.num_key_value_heads

    def kv_bytes_per_token(self, dtype: str = "bf16") -> int:
        """Bytes of K and V that one token holds over all layers (layover/config.py:98-102)."""
        return self.num_hidden_layers * 2 * self.num_key_value_heads * self.head_dim * DTYPE_BYTES[dtype]


# Named shapes for the command line and the benchmark. These are inputs a user may choose
# instead of a model folder, not constants of the engine: every one goes through
# `Qwen3Config(...)` like a parsed config.json.
PRESETS: dict[str, dict] = {
    "tiny-a": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                   max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                   tie_word_embeddings=True),
    "tiny-b": dict(vocab_size=512, hidden_size=96, intermediate_size=200, num_hidden_layers=3,
                   num_attention_heads=6, num_key_value_heads=1, head_dim=32,
                   max_position_embeddings=512, rope_theta=1000000.0, rms_norm_eps=1e-5,
                   tie_word_embeddings=False),
    "qwen3-4b": dict(vocab_size=151936, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                     num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6,
                     tie_word_embeddings=True),
    "qwen3-8b": dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                     num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6,
                     tie_word_embeddings=False),
    "qwen3-32b": dict(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                      num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                      max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6,
                      tie_word_embeddings=False),
}


def preset(name: str, **overrides) -> Qwen3Config:
    if name not in PRESETS:
        raise ValueError(f"unknown preset {name!r}; known: {sorted(PRESETS)}")
    return Qwen3Config(**{**PRESETS[name], **overrides})
