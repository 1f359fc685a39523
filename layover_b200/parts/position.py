"""Position encodings that a mixer applies to its queries and keys."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, register_position


@register_position("rotary_half")
class RotaryHalf(Part):
    """Rotary embedding over the whole head, pairing lane i with lane i + dim/2.

    inv_freq[i] = theta^(-2i/dim) in 32-bit (layover/model.py:185); angle = position * inv_freq;
    x' = x cos + rotate_half(x) sin (layover/model.py:100-102,127-128). The frequencies are made once
    at build time; `tables(batch)` makes the step's cos/sin table [T, 2, dim/2] in 32-bit once per
    step (every layer with the same head size and theta shares it, as the reference computes its
    tables once per call, layover/model.py:220-221); the rotation itself runs inside the mixer's
    fused kernel.

    params: dim (the head's size), theta."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("dim", "theta")
        self.dim, self.theta = int(params["dim"]), float(params["theta"])
        if self.dim % 2:
            raise ValueError("rotary_half needs an even head size")
        self._table = None

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        exponent = torch.arange(0, self.dim, 2, dtype=torch.float32) / self.dim
        self._table = (1.0 / (self.theta ** exponent)).to(runtime.device).contiguous()

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def inv_freq(self) -> torch.Tensor:
        return self._table

    def tables(self, batch) -> torch.Tensor | None:
        """The step's cos/sin table for the fused kernel; parts that cannot be fused return None."""
        key = ("rotary_half", self.dim, self.theta)
        table = batch.shared.get(key)
        if table is None:
            table = torch.empty((batch.n_tokens, 2, self.dim // 2), dtype=torch.float32, device=self._table.device)
            ops.rope_table(batch.positions, self._table, table)
            batch.shared[key] = table
        return table

    def apply(self, q, k, positions):  # only reached when a mixer cannot fuse the rotation
        raise NotImplementedError("rotary_half runs inside the mixer's fused kernel")
