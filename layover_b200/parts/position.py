"""Position encodings that a mixer applies to its queries and keys."""

from __future__ import annotations

import torch

from .base import Part, register_position


@register_position("rotary_half")
class RotaryHalf(Part):
    """Rotary embedding over the whole head, pairing lane i with lane i + dim/2.

    inv_freq[i] = theta^(-2i/dim) in 32-bit (layover/model.py:185); angle = position * inv_freq;
    x' = x cos + rotate_half(x) sin (layover/model.py:100-102,127-128). The table is made once at
    build time; the rotation itself runs inside the mixer's fused kernel, which asks for the
    table through `inv_freq`.

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

    def inv_freq(self) -> torch.Tensor | None:
        return self._table

    def apply(self, q, k, positions):  # only reached when a mixer cannot fuse the rotation
        raise NotImplementedError("rotary_half runs inside the mixer's fused kernel")
