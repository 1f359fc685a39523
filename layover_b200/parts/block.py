"""Arrangements of a layer's parts."""

from __future__ import annotations

from .. import profiling
from .base import Part, build_part, register_block


@register_block("pre_norm")
class PreNormBlock(Part):
    """x = x + mixer(norm(x)); x = x + feed_forward(norm(x)) (layover/model.py:164-166,224).

    The additions are not launched here: each sub-layer's output is handed on as `delta` and the
    next norm (of this block, of the next block, or the model's final norm) adds it into the
    residual stream before normalising.

    params: input_norm, mixer, post_norm, feed_forward (PartSpecs)."""

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("input_norm", "mixer", "post_norm", "feed_forward")
        self.input_norm = build_part("norm", params["input_norm"], prefix)
        self.mixer = build_part("mixer", params["mixer"], prefix)
        self.post_norm = build_part("norm", params["post_norm"], prefix)
        self.feed_forward = build_part("feed_forward", params["feed_forward"], prefix)

    def parts(self):
        return [self.input_norm, self.mixer, self.post_norm, self.feed_forward]

    def tensor_specs(self):
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for part in self.parts():
            part.bind(tensors, runtime)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, delta, batch, cache):
        if profiling.active():
            with profiling.nvtx_range("mixer"):
                h = self.input_norm.forward(x, delta)
                attended = self.mixer.forward(h, batch, cache)
            with profiling.nvtx_range("feed_forward"):
                h = self.post_norm.forward(x, attended)
                return x, self.feed_forward.forward(h)
        h = self.input_norm.forward(x, delta)
        attended = self.mixer.forward(h, batch, cache)
        h = self.post_norm.forward(x, attended)
        return x, self.feed_forward.forward(h)
