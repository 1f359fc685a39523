"""The run's precision: which matrix product and which attention kernels the parts call.

float32 is the true 32-bit path: FFMA products, one 32-bit attention kernel for every segment
length, nothing in reduced precision. bfloat16 is the serving path: tensor-core products and
attention with 32-bit accumulation and softmax. There is no other backend behind either.
"""

from __future__ import annotations

import torch

from .. import ops
from ..parts.base import Runtime


def _linear_f32(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    out = torch.empty((a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
    return ops.gemm_simt(a, w, out)


def _linear_bf16(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype or torch.bfloat16, device=a.device)
    return ops.gemm_bf16(a, w, out)


def _linear_swiglu_bf16(a: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor | None:
    """silu(a Wg^T) * (a Wu^T) over interleaved weights. Many tokens, or at most 16: one product with
    the activation in its epilogue (the [T, 2 I] tensor is never written). In between: product, then
    the activation kernel, which is faster there (measured for a whole feed-forward at 64 tokens:
    41.7 us against 43.5 us fused; in a decode step of 8 sequences the fused product takes 0.05 ms
    off 3.06 ms)."""
    tokens, inter = a.shape[0], w_interleaved.shape[0] // 2
    out = torch.empty((tokens, inter), dtype=torch.bfloat16, device=a.device)
    if (tokens > 128 or tokens <= 16) and ops.gemm_tcgen05_supports(a, w_interleaved):
        return ops.gemm_tcgen05(a, w_interleaved, out, epilogue="swiglu")
    gate_up = torch.empty((tokens, 2 * inter), dtype=torch.bfloat16, device=a.device)
    ops.gemm_bf16(a, w_interleaved, gate_up)
    return ops.swiglu(gate_up, out, block=ops.SWIGLU_BLOCK)


def _attention_simt(q, cache, out, block_table, batch, q_heads, kv_heads, dim, page_tokens, scale, window):
    tiles = batch.tiles[ops.attention_simt_block_queries()]
    ops.attention_simt(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, tiles.tile_seq, tiles.tile_q0,
                       tiles.count, q_heads, kv_heads, dim, page_tokens, scale, window)


def make_runtime(dtype: torch.dtype, device: torch.device | str) -> Runtime:
    device = torch.device(device)
    if device.type != "cuda":
        raise ops.KernelError("layover_b200 runs on a CUDA device only: there is no CPU path")
    if dtype == torch.float32:
        runtime = Runtime(dtype, device, _linear_f32)
        runtime.attention = _attention_simt
        runtime.tile_sizes = (ops.attention_simt_block_queries(),)
        runtime.kernel_libraries = ("elementwise", "gemm_simt", "attention_simt", "sampling")
    elif dtype == torch.bfloat16:
        ops.gemm_scratch(device)      # made now, never inside a graph capture
        ops.attention_scratch(device)
        runtime = Runtime(dtype, device, _linear_bf16)
        runtime.attention = ops.attention_bf16
        runtime.linear_swiglu = _linear_swiglu_bf16
        runtime.linear_heads = ops.gemm_qkv_heads
        runtime.swiglu_block = ops.SWIGLU_BLOCK
        runtime.interleave_gate_up = ops.interleave_gate_up
        runtime.tile_sizes = ops.attention_bf16_tile_sizes()
        runtime.kernel_libraries = ops.BF16_LIBRARIES
    else:
        raise ValueError(f"unsupported dtype {dtype}; the engine runs float32 or bfloat16")
    return runtime
