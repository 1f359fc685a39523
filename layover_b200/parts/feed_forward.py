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
    product reads x once. Where the run's precision offers a product with the activation in its
    epilogue (and the width allows it), the rows are interleaved for it and no [T, 2 inter]
    tensor is ever written; otherwise the activation kernel reads both halves of its row."""

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
        self.fused = (runtime.linear_swiglu is not None and runtime.swiglu_block > 0
                      and self.inter % runtime.swiglu_block == 0)
        if self.fused:
            self.gate_up = runtime.interleave_gate_up(gate, up)
        else:
            self.gate_up = torch.cat((gate, up), dim=0).contiguous()
        self.down = tensors[self.names["down"]]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return self.runtime.linear(self.runtime.linear_swiglu(h, self.gate_up), self.down)
        gate_up = self.runtime.linear(h, self.gate_up)
        act = torch.empty((h.shape[0], self.inter), dtype=h.dtype, device=h.device)
        ops.swiglu(gate_up, act)
        return self.runtime.linear(act, self.down)
