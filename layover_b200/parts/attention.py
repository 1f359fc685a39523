"""Grouped-query attention over the paged cache."""

from __future__ import annotations

import math

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import PagedKVNeed, Part, PartSpec, build_part, register_mixer


@register_mixer("attention")
class Attention(Part):
    """q/k/v projections without bias, optional per-head RMSNorm of q and k, a position encoding,
    keys and values written to their pages, causal attention over the block table with scale
    1/sqrt(head_dim), output projection (layover/model.py:105-142).

    params: hidden, q_heads, kv_heads, head_dim; qk_norm_eps (None: no per-head norm);
    position (a PartSpec or None); window (None: every earlier key is seen);
    shares_cache (True: the layer has no k/v projections and attends over another layer's
    pages); tensor names q, k, v, o (and q_norm, k_norm with a per-head norm) relative to the
    prefix: the architecture's spec gives them, the part knows no checkpoint's naming.

    Kernels are chosen when the part is bound: a float32 run attends with the one 32-bit kernel
    for every segment length; a bfloat16 run with the tensor-core kernels (tcgen05 tiles where
    they take the head size, mma.sync tiles elsewhere, the split decode kernel for single
    tokens) and, for steps of few tokens, a q/k/v product with norm, rotation and page write in
    its epilogue.

    The three projections are stacked at load into one [(q_heads + 2 kv_heads) head_dim, hidden]
    matrix (the reference runs three products, layover/model.py:121-123)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "q_heads", "kv_heads", "head_dim")
        p = params
        self.hidden, self.q_heads, self.kv_heads, self.dim = (int(p[k]) for k in ("hidden", "q_heads", "kv_heads", "head_dim"))
        if self.q_heads % self.kv_heads:
            raise ValueError(f"q_heads ({self.q_heads}) must be divisible by kv_heads ({self.kv_heads})")
        if self.dim % 16:
            raise ValueError(f"head_dim must be a multiple of 16, got {self.dim}")
        if self.dim > 256:
            raise ValueError(f"head_dim up to 256 is supported, got {self.dim}")
        self.qk_norm_eps = p.get("qk_norm_eps")
        self.window = p.get("window")
        self.shares_cache = bool(p.get("shares_cache", False))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.dim)))
        self.position = build_part("position", p.get("position"), prefix)
        wanted = ["q", "o"] + ([] if self.shares_cache else ["k", "v"])
        if self.qk_norm_eps is not None:
            wanted += ["q_norm"] + ([] if self.shares_cache else ["k_norm"])
        self.require(*wanted)
        self.names = {k: prefix + p[k] for k in wanted}
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        self._attend = self._project_heads = None

    # ---- what it wants
    def tensor_specs(self):
        n = self.names
        specs = [TensorSpec(n["q"], (self.q_heads * self.dim, self.hidden))]
        if not self.shares_cache:
            specs += [TensorSpec(n["k"], (self.kv_heads * self.dim, self.hidden)),
                      TensorSpec(n["v"], (self.kv_heads * self.dim, self.hidden))]
        specs.append(TensorSpec(n["o"], (self.hidden, self.q_heads * self.dim)))
        if self.qk_norm_eps is not None:
            specs.append(TensorSpec(n["q_norm"], (self.dim,), kind="vector", init="ones"))
            if not self.shares_cache:
                specs.append(TensorSpec(n["k_norm"], (self.dim,), kind="vector", init="ones"))
        if self.position is not None:
            specs += self.position.tensor_specs()
        return specs

    def cache_need(self):
        return PagedKVNeed(self.kv_heads, self.dim, self.window)

    def parts(self):
        return [self.position] if self.position is not None else []

    def kernel_libraries(self, dtype):
        if dtype == torch.float32:
            return ("elementwise", "attention_simt")
        names = ["elementwise", "attention_mma"]
        if ops.attention_tcgen05_takes_heads(self.q_heads, self.kv_heads, self.dim):
            names.append("attention_tcgen05")
        return tuple(names)

    def tile_sizes(self, dtype):
        if dtype == torch.float32:
            return (ops.attention_simt_block_queries(),)
        sizes = [ops.attention_mma_block_queries()]
        if ops.attention_tcgen05_takes_heads(self.q_heads, self.kv_heads, self.dim):
            sizes.append(ops.TCGEN05_TILE)
        return tuple(sizes)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        if runtime.dtype == torch.float32:
            self._attend, self._project_heads = ops.attention_f32, None
        else:
            ops.attention_scratch(runtime.device)      # made now, never inside a graph capture
            self._attend, self._project_heads = ops.attention_bf16, ops.gemm_qkv_heads
        n = self.names
        if self.shares_cache:
            self.w_qkv = tensors[n["q"]]
        else:
            self.w_qkv = torch.cat((tensors.pop(n["q"]), tensors.pop(n["k"]), tensors.pop(n["v"])), dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.qk_norm_eps is not None:
            self.q_norm_w = tensors[n["q_norm"]]
            self.k_norm_w = None if self.shares_cache else tensors[n["k_norm"]]
        if self.position is not None:
            self.position.bind(tensors, runtime)

    # ---- one step
    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        q = self.project(h, batch, cache)
        out = torch.empty_like(q)
        self.attend(q, cache, batch, batch.groups[cache.group], out)
        return self.runtime.linear(out, self.w_o)

    def project(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        """q [T, q_heads * head_dim], normed and rotated; this step's keys and values go to their pages."""
        tokens = h.shape[0]
        own_kv = 0 if self.shares_cache else self.kv_heads
        group = batch.groups[cache.group]
        q = torch.empty((tokens, self.q_heads * self.dim), dtype=h.dtype, device=h.device)
        eps = float(self.qk_norm_eps or 0.0)
        table = self.position.tables(batch) if self.position is not None else None
        fused = self.position is None or table is not None
        k_pool, v_pool = (cache.k_pool, cache.v_pool) if own_kv else (None, None)
        heads = self._project_heads
        if (heads is not None and own_kv and table is not None and self.qk_norm_eps is not None
                and heads(h, self.w_qkv, q, k_pool, v_pool, self.q_norm_w, self.k_norm_w, table, group.slot_map,
                          self.q_heads, own_kv, self.dim, cache.page_tokens, eps)):
            return q                       # projection, norm, rotation and page write were one kernel
        qkv = self.runtime.linear(h, self.w_qkv)
        if fused:
            ops.qk_norm_rope_kv(qkv, q, k_pool, v_pool, self.q_norm_w, self.k_norm_w, table, group.slot_map,
                                self.q_heads, own_kv, self.dim, cache.page_tokens, eps)
        else:
            # norm in place, the position encoding as its own step, then the page write
            ops.qk_norm_rope_kv(qkv, q, None, None, self.q_norm_w, self.k_norm_w, None, None,
                                self.q_heads, own_kv, self.dim, cache.page_tokens, eps)
            k_rows = qkv[:, self.q_heads * self.dim:(self.q_heads + own_kv) * self.dim]
            self.position.apply(q.view(tokens, self.q_heads, self.dim),
                                k_rows.unflatten(1, (own_kv, self.dim)) if own_kv else None, batch.positions)
            if own_kv:
                ops.qk_norm_rope_kv(qkv, None, k_pool, v_pool, None, None, None, group.slot_map,
                                    self.q_heads, own_kv, self.dim, cache.page_tokens, eps)
        return q

    def attend(self, q, cache, batch, group, out) -> None:
        self._attend(q, cache, out, group.block_table, batch, self.q_heads, self.kv_heads, self.dim,
                     cache.page_tokens, self.scale, self.window or 0)


def attention_spec(hidden, q_heads, kv_heads, head_dim, qk_norm_eps, theta, names: dict[str, str], window=None,
                   shares_cache=False) -> PartSpec:
    """`names`: the checkpoint's tensor names for q, k, v, o, q_norm, k_norm, relative to the layer's prefix."""
    position = PartSpec("rotary_half", {"dim": head_dim, "theta": theta}) if theta is not None else None
    return PartSpec("attention", {
        "hidden": hidden, "q_heads": q_heads, "kv_heads": kv_heads, "head_dim": head_dim,
        "qk_norm_eps": qk_norm_eps, "position": position, "window": window, "shares_cache": shares_cache, **names,
    })
