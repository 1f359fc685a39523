"""A plain, slow Qwen3 dense forward pass used as the oracle of the test-suite.

Whole sequences, no cache, one function for each part. It shares no code with the
package under test: it parses config.json itself, takes weights as a plain dict of
tensors by checkpoint name, and computes everything with elementary torch ops on
the CPU. Every function cites the lines of CarlGergi/Layover (paths inside that
project) whose formula it restates.

`tests/golden/make_golden.py` compared this file once with the reference's own
model code on a tiny random model; `tests/test_plain.py` checks this file against
the outputs committed by that script.

Two extras that the reference does not have are kept here only so that toy parts in
the tests have an oracle: an optional attention window and a layer schedule that may
repeat a layer or let a layer attend over another layer's keys and values.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def plain_config(raw: dict) -> dict:
    """Sizes and constants, with the reference's defaults (layover/config.py:28-59)."""
    if raw.get("model_type", "qwen3") != "qwen3":
        raise ValueError("not a qwen3 config")
    rope = raw.get("rope_parameters") or raw.get("rope_scaling") or {}
    heads = raw["num_attention_heads"]
    return {
        "vocab": raw["vocab_size"],
        "hidden": raw["hidden_size"],
        "inter": raw["intermediate_size"],
        "layers": raw["num_hidden_layers"],
        "heads": heads,
        "kv_heads": raw.get("num_key_value_heads") or heads,
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads,
        "theta": float(raw.get("rope_theta", rope.get("rope_theta", 10000.0))),
        "eps": raw.get("rms_norm_eps", 1e-6),
        "tied": raw.get("tie_word_embeddings", True),
    }


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Variance in 32-bit, rounded to x's dtype, then times the weight (layover/model.py:31-36)."""
    wide = x.float()
    scaled = wide * torch.rsqrt(wide.pow(2).mean(-1, keepdim=True) + eps)
    return weight.to(x.dtype) * scaled.to(x.dtype)


def plain_rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype):
    """cos and sin [tokens, head_dim]: angles in 32-bit, the two halves alike, rounded to dtype
    (layover/model.py:185 for the frequencies, layover/model.py:193-197 for the tables)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    angles = positions.float()[:, None] * inv_freq[None, :]
    angles = torch.cat((angles, angles), dim=-1)
    return angles.cos().to(dtype), angles.sin().to(dtype)


def plain_rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(-right half, left half) (layover/model.py:100-102)."""
    left, right = x.chunk(2, dim=-1)
    return torch.cat((-right, left), dim=-1)


def plain_apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [tokens, heads, dim]; x*cos + rotate_half(x)*sin in x's dtype (layover/model.py:127-128)."""
    return x * cos[:, None, :] + plain_rotate_half(x) * sin[:, None, :]


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [tokens, heads, dim], k and v [tokens, kv_heads, dim]; query head h reads KV head
    h // (heads // kv_heads); scale 1/sqrt(dim); query t sees keys j <= t
    (layover/model.py:59 for the mask, :90-96 for the scale and grouping,
    layover/kernels/triton_decode.py:95-115 for softmax and sums in 32-bit).
    With `window`, key j is seen only if t - j < window (not in the reference).
    """
    tokens, heads, dim = q.shape
    groups = heads // k.shape[1]
    qf, kf, vf = q.float(), k.float(), v.float()
    t = torch.arange(tokens)
    allowed = t[None, :] <= t[:, None]
    if window is not None:
        allowed &= (t[:, None] - t[None, :]) < window
    out = torch.empty(tokens, heads, dim, dtype=torch.float32)
    for h in range(heads):
        scores = (qf[:, h] @ kf[:, h // groups].T) / math.sqrt(dim)
        scores = scores.masked_fill(~allowed, float("-inf"))
        out[:, h] = torch.softmax(scores, dim=-1) @ vf[:, h // groups]
    return out.to(q.dtype)


def plain_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x W^T, no bias (layover/model.py:110-113,148-150,182)."""
    return x @ weight.T


def plain_mlp(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (layover/model.py:152-153)."""
    return plain_linear(torch.nn.functional.silu(plain_linear(x, gate)) * plain_linear(x, up), down)


def plain_qkv(x, weights, prefix, cfg, positions):
    """q, k, v of one layer after per-head norm and rotation (layover/model.py:117-129)."""
    tokens = x.shape[0]
    dim = cfg["head_dim"]
    q = plain_linear(x, weights[prefix + "self_attn.q_proj.weight"]).view(tokens, cfg["heads"], dim)
    k = plain_linear(x, weights[prefix + "self_attn.k_proj.weight"]).view(tokens, cfg["kv_heads"], dim)
    v = plain_linear(x, weights[prefix + "self_attn.v_proj.weight"]).view(tokens, cfg["kv_heads"], dim)
    q = plain_rmsnorm(q, weights[prefix + "self_attn.q_norm.weight"], cfg["eps"])
    k = plain_rmsnorm(k, weights[prefix + "self_attn.k_norm.weight"], cfg["eps"])
    cos, sin = plain_rope_tables(positions, dim, cfg["theta"], x.dtype)
    return plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin), v


def plain_block(x, weights, layer: int, cfg, positions, window=None, shared_kv=None):
    """One decoder layer: x + attn(norm(x)), then + mlp(norm(.)) (layover/model.py:164-166,224).

    Returns the new x and this layer's (k, v). With `shared_kv`, the layer attends over
    those keys and values instead of its own (not in the reference)."""
    prefix = f"model.layers.{layer}."
    h = plain_rmsnorm(x, weights[prefix + "input_layernorm.weight"], cfg["eps"])
    q, k, v = plain_qkv(h, weights, prefix, cfg, positions)
    if shared_kv is not None:
        k, v = shared_kv
    attended = plain_attention(q, k, v, window).reshape(x.shape[0], -1)
    x = x + plain_linear(attended, weights[prefix + "self_attn.o_proj.weight"])
    h = plain_rmsnorm(x, weights[prefix + "post_attention_layernorm.weight"], cfg["eps"])
    x = x + plain_mlp(
        h,
        weights[prefix + "mlp.gate_proj.weight"],
        weights[prefix + "mlp.up_proj.weight"],
        weights[prefix + "mlp.down_proj.weight"],
    )
    return x, (k, v)


def plain_forward(
    raw_config: dict,
    weights: dict[str, torch.Tensor],
    tokens,
    dtype: torch.dtype = torch.float32,
    window: int | None = None,
    schedule: list[tuple[int, int | None]] | None = None,
) -> torch.Tensor:
    """Logits [tokens, vocab] in 32-bit for one whole sequence (layover/model.py:199-230).

    `weights` holds the checkpoint's tensors by name; they are cast to `dtype` as the
    reference does at load (layover/weights.py:33-35). `schedule` lists (layer, index of an
    earlier schedule entry whose keys and values to read, or None); by default every layer
    runs once in order with its own keys and values.
    """
    cfg = plain_config(raw_config)
    w = {name: t.to(dtype) if t.is_floating_point() else t for name, t in weights.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    x = w["model.embed_tokens.weight"][ids]
    schedule = schedule or [(i, None) for i in range(cfg["layers"])]
    kept = []
    for layer, reads in schedule:
        x, kv = plain_block(x, w, layer, cfg, positions, window, None if reads is None else kept[reads])
        kept.append(kv)
    x = plain_rmsnorm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return plain_linear(x, head).float()


# --- sampling -------------------------------------------------------------------------

PHILOX_M0, PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
PHILOX_W0, PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def plain_philox4x32(counter: np.ndarray, key: tuple[int, int]) -> np.ndarray:
    """Philox-4x32 with 10 rounds (Salmon et al., SC 2011) over counters [n, 4] of uint32.

    The reference samples greedily only (layover/engine.py:139-141); temperature sampling is
    defined by this function and `plain_sample`.
    """
    c = counter.astype(np.uint64)
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(PHILOX_M0) * c[:, 0]
        p1 = np.uint64(PHILOX_M1) * c[:, 2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = np.stack([(hi1 ^ c[:, 1] ^ k0) & mask, lo1, (hi0 ^ c[:, 3] ^ k1) & mask, lo0], axis=1)
        k0 = (k0 + np.uint64(PHILOX_W0)) & mask
        k1 = (k1 + np.uint64(PHILOX_W1)) & mask
    return c.astype(np.uint32)


def plain_uniform(seed: int, step: int, vocab: int) -> np.ndarray:
    """One uniform in (0, 1) for each vocabulary entry of one request's `step`-th sampled token.

    Counter = (entry // 4, step, 0, 0), key = the seed's low and high words; entry v takes word
    v % 4 of its block; u = (word + 0.5) / 2^32 computed in 32-bit floats."""
    blocks = (vocab + 3) // 4
    counter = np.zeros((blocks, 4), dtype=np.uint32)
    counter[:, 0] = np.arange(blocks, dtype=np.uint32)
    counter[:, 1] = np.uint32(step)
    words = plain_philox4x32(counter, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)).reshape(-1)[:vocab]
    # 24 high bits, so that the float is exact and strictly inside (0, 1)
    return ((words >> np.uint32(8)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0**-24)


def plain_sample(logits: np.ndarray, temperature: float, seed: int, step: int) -> int:
    """Greedy for temperature 0 (first of equal maxima, layover/engine.py:141); otherwise the
    Gumbel-max draw argmax(logits / T - log(-log(u)))."""
    logits = np.asarray(logits, dtype=np.float32)
    if temperature == 0.0:
        return int(np.argmax(logits))
    u = plain_uniform(seed, step, logits.shape[0])
    gumbel = -np.log(-np.log(u.astype(np.float64)))
    return int(np.argmax(logits.astype(np.float64) / np.float64(np.float32(temperature)) + gumbel))


def plain_generate(raw_config, weights, prompt, steps, dtype=torch.float32, temperature=0.0, seed=0):
    """Generate `steps` tokens by running the whole sequence again for every token."""
    tokens = list(prompt)
    out = []
    for step in range(steps):
        logits = plain_forward(raw_config, weights, tokens, dtype)[-1].numpy()
        token = plain_sample(logits, temperature, seed, step)
        out.append(token)
        tokens.append(token)
    return out
