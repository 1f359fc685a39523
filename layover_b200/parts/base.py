"""The kinds of parts a layer is put together from, their interfaces and their registries.

A model is a list of layers; a layer is a *block* (an arrangement) of a *mixer* (attention
here), a *feed-forward* and *norms*; a mixer may use a *position encoding*. Each part is built
from a `PartSpec`: the registered name of its kind and its sizes and constants as parameters.
No part knows which model it is in. A new kind is one class and one `register_*` call; the
model spec of an architecture then names it, layer by layer.

What each kind must offer:

  every part      tensor_specs() -> [TensorSpec]      the checkpoint tensors it wants
                  bind(tensors, runtime)              take them (fuse or reshape as it likes)
  norm            forward(x, delta, rows=None) -> h   x += delta in place (delta may be None), h = norm(x);
                                                      with rows, only those rows, x untouched
  position        tables(batch) -> float32 [T, 2, dim/2] cos/sin of the step, or None; made once per
                                                      step and kept in batch.shared (the fused kernel applies it)
                  apply(q, k, positions)              when tables() is None: rotate q [T, heads, dim], k in place
  mixer           cache_need() -> PagedKVNeed | StateNeed | None
                  forward(h, batch, cache) -> [T, hidden]     cache is the view it was given for its need
  feed-forward    forward(h) -> [T, hidden]
  block           forward(x, delta, batch, cache) -> (x, delta)   the residual stream and the
                                                      not-yet-added output of the last sub-layer
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token (window None) or of the last `window` tokens, in pages."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per live request, zeroed when the request starts."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What a part needs to know about the run: precision, device and the matrix product."""
    dtype: torch.dtype
    device: torch.device
    linear: Callable[..., torch.Tensor]   # linear(a [M, K], w [N, K], out_dtype=None) -> [M, N]
    # attention(q, cache_view, out, block_table, batch, q_heads, kv_heads, dim, page_tokens, scale, window)
    attention: Callable[..., None] | None = None
    # linear_swiglu(a, w_interleaved) -> silu(gate) * up or None; w made by interleave_gate_up(gate, up)
    linear_swiglu: Callable[..., torch.Tensor | None] | None = None
    interleave_gate_up: Callable[..., torch.Tensor] | None = None
    # linear_heads(h, w_qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, table, slot_map, q_heads, kv_heads, dim,
    #              page_tokens, eps) -> bool: the stacked q/k/v projection with the per-head norm, the rotation
    #              and the page write in its epilogue; False (nothing done) where the run or the sizes have none
    linear_heads: Callable[..., bool] | None = None
    swiglu_block: int = 0                 # the fused product wants the width to be a multiple of this
    tile_sizes: tuple[int, ...] = ()      # query-tile sizes whose tile lists the batch must carry
    kernel_libraries: tuple[str, ...] = ()  # what has to be compiled before the first step


class Part:
    def __init__(self, params: dict, prefix: str):
        self.params = dict(params)
        self.prefix = prefix

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime

    def require(self, *names: str) -> None:
        missing = [n for n in names if n not in self.params]
        if missing:
            raise ValueError(f"{type(self).__name__} lacks parameters {missing}")


_REGISTRIES: dict[str, dict[str, type]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {}}


def _register(family: str, kind: str, cls: type | None = None):
    def put(c):
        _REGISTRIES[family][kind] = c
        return c
    return put(cls) if cls is not None else put


def register_norm(kind: str, cls: type | None = None):
    return _register("norm", kind, cls)


def register_position(kind: str, cls: type | None = None):
    return _register("position", kind, cls)


def register_mixer(kind: str, cls: type | None = None):
    return _register("mixer", kind, cls)


def register_feed_forward(kind: str, cls: type | None = None):
    return _register("feed_forward", kind, cls)


def register_block(kind: str, cls: type | None = None):
    return _register("block", kind, cls)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def registered(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])


def build_part(family: str, spec: PartSpec | None, prefix: str, **extra: Any):
    """Instantiate the part that `spec` names from its family's registry."""
    if spec is None:
        return None
    try:
        cls = _REGISTRIES[family][spec.kind]
    except KeyError:
        raise ValueError(f"unknown {family} kind {spec.kind!r}; registered: {registered(family)}") from None
    return cls(spec.params, prefix, **extra)
