"""RMSNorm, fused with the residual addition that precedes it."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    """y = weight * round(x * rsqrt(mean(x^2) + eps)), statistics in 32-bit (layover/model.py:25-36).

    params: dim, eps, weight (tensor name relative to the prefix).
    `forward(x, delta)` first adds `delta` into `x` (the residual sum, in 32-bit, rounded once)
    so that a block never launches a separate addition."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("dim", "eps", "weight")
        self.dim, self.eps = int(params["dim"]), float(params["eps"])
        self.weight_name = prefix + params["weight"]
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.dim,), kind="vector", init="ones")]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.weight_name]

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor | None = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.dim), dtype=x.dtype, device=x.device)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
