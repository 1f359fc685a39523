"""Qwen3 dense as a list of layers (layover/model.py:156-186): every layer is a pre-norm block of
grouped-query attention with per-head RMSNorm of q and k and rotary embedding over the whole head,
and a SiLU-gated feed-forward; RMSNorm everywhere with one eps; the output matrix may be the
embedding. Tensor names are the checkpoint's own (layover/model.py:3)."""

from __future__ import annotations

from ..config.base import register_architecture
from ..config.qwen3 import Qwen3Config
from ..parts.attention import attention_spec
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    def norm(weight: str, dim: int) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": dim, "eps": cfg.rms_norm_eps, "weight": weight})

    attention_names = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight",
                       "o": "self_attn.o_proj.weight", "q_norm": "self_attn.q_norm.weight",
                       "k_norm": "self_attn.k_norm.weight"}
    layers = []
    for index in range(cfg.num_hidden_layers):
        block = PartSpec("pre_norm", {
            "input_norm": norm("input_layernorm.weight", cfg.hidden_size),
            "mixer": attention_spec(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                    qk_norm_eps=cfg.rms_norm_eps, theta=cfg.rope_theta, names=attention_names),
            "post_norm": norm("post_attention_layernorm.weight", cfg.hidden_size),
            "feed_forward": PartSpec("gated_mlp", {
                "hidden": cfg.hidden_size, "inter": cfg.intermediate_size, "activation": "silu",
                "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"}),
        })
        layers.append(LayerSpec(block, f"model.layers.{index}."))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_position=cfg.max_position_embeddings,
        embedding="model.embed_tokens.weight",
        final_norm=norm("model.norm.weight", cfg.hidden_size),
        head=None if cfg.tie_word_embeddings else "lm_head.weight",
        layers=layers,
        # a tied checkpoint may still carry a copy of the head (layover/weights.py:36-37)
        ignorable_tensors=frozenset({"lm_head.weight"}) if cfg.tie_word_embeddings else frozenset(),
    )


register_architecture(Qwen3Config.architecture, Qwen3Config.model_type, Qwen3Config, qwen3_spec)
