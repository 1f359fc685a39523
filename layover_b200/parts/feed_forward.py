"""Feed-forward parts."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Part, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    """down(act(gate(x)) * up(x)) without bias (layover/model.py:145-153); act = silu.

    params: hidden, inter, activation ("silu"), gate, up, down (tensor names relative to the
    prefix). gate and up are stacked at load into one [2 inter, hidden] matrix so that one
    product reads x once. In a bfloat16 run whose width allows it, the rows are interleaved for
    the tensor-core product with the activation in its epilogue and no [T, 2 inter] tensor is ever
    written; otherwise the activation kernel reads both halves of its row."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("hidden", "inter", "gate", "up", "down")
        self.hidden, self.inter = int(params["hidden"]), int(params["inter"])
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: unsupported activation {params['activation']!r}")
        self.names = {k: prefix + params[k] for k in ("gate", "up", "down")}
        self.gate_up = self.down = None

    def tensor_specs(self):
        return [
            TensorSpec(self.names["gate"], (self.inter, self.hidden)),
            TensorSpec(self.names["up"], (self.inter, self.hidden)),
            TensorSpec(self.names["down"], (self.hidden, self.inter)),
        ]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        gate, up = tensors.pop(self.names["gate"]), tensors.pop(self.names["up"])
        self.fused = runtime.dtype == torch.bfloat16 and self.inter % ops.SWIGLU_BLOCK == 0
        if self.fused:
            self.gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.gate_up = torch.cat((gate, up), dim=0).contiguous()
        self.down = tensors[self.names["down"]]

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def activated(self, h: torch.Tensor) -> torch.Tensor:
        """silu(h Wg^T) * (h Wu^T) over the interleaved weights. Many tokens, or at most 16: one
        product with the activation in its epilogue. In between: product, then the activation kernel,
        which is faster there (a whole feed-forward at 64 tokens: 41.7 us against 43.5 us fused)."""
        tokens = h.shape[0]
        out = torch.empty((tokens, self.inter), dtype=torch.bfloat16, device=h.device)
        if (tokens > 128 or tokens <= 16) and ops.gemm_tcgen05_supports(h, self.gate_up):
            return ops.gemm_tcgen05(h, self.gate_up, out, epilogue="swiglu")
        gate_up = self.runtime.linear(h, self.gate_up)
        return ops.swiglu(gate_up, out, block=ops.SWIGLU_BLOCK)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return self.runtime.linear(self.activated(h), self.down)
        gate_up = self.runtime.linear(h, self.gate_up)
        act = torch.empty((h.shape[0], self.inter), dtype=h.dtype, device=h.device)
        ops.swiglu(gate_up, act)
        return self.runtime.linear(act, self.down)
