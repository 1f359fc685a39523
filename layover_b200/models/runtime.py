"""The run's precision and its matrix product.

float32 is the true 32-bit path: FFMA products, nothing in reduced precision. bfloat16 is the
serving path: tensor-core products with 32-bit accumulation. There is no other backend behind
either. Everything beyond the plain product (attention kernels, fused epilogues) is chosen by
the parts themselves when they are bound (`Part.bind`), from `Runtime.dtype`.
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


def make_runtime(dtype: torch.dtype, device: torch.device | str) -> Runtime:
    device = torch.device(device)
    if device.type != "cuda":
        raise ops.KernelError("layover_b200 runs on a CUDA device only: there is no CPU path")
    if dtype == torch.float32:
        return Runtime(dtype, device, _linear_f32, kernel_libraries=("gemm_simt",))
    if dtype == torch.bfloat16:
        ops.gemm_scratch(device)      # made now, never inside a graph capture
        return Runtime(dtype, device, _linear_bf16, kernel_libraries=("gemm_simt", "gemm_tcgen05"))
    raise ValueError(f"unsupported dtype {dtype}; the engine runs float32 or bfloat16")
