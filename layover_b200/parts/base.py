"""The kinds of parts a layer is put together from, their interfaces and their registries.

A model is a list of layers; a layer is a *block* (an arrangement) of a *mixer* (attention
here), a *feed-forward* and *norms*; a mixer may use a *position encoding*. Each part is built
from a `PartSpec`: the registered name of its kind and its sizes and constants as parameters.
No part knows which model it is in. A new kind is one class and one `register_*` call; the
model spec of an architecture then names it, layer by layer.

What each kind must offer:

  every part      tensor_specs() -> [TensorSpec]      the checkpoint tensors it wants
                  bind(tensors, runtime)              take them (fuse or reshape as it likes) and choose
                                                      its kernels for runtime.dtype
                  parts() -> [Part]                   its own sub-parts (default: none)
                  kernel_libraries(dtype) -> names    kernel libraries it launches (default: none)
                  tile_sizes(dtype) -> sizes          query-tile lists it wants in a batch (default: none)
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

    def elements_per_token(self) -> int:
        """Pool elements one token takes in one layer with this need (keys and values)."""
        return 2 * self.kv_heads * self.head_dim


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per live request, zeroed when the request starts."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What a part needs to know about the run: its precision, its device and the matrix product
    of that precision. Everything else (which attention kernel, which fused product) a part
    chooses for itself from `dtype` when it is bound; `extras` carries whatever else a caller
    wants its own parts to find (the package's parts read nothing from it)."""
    dtype: torch.dtype
    device: torch.device
    linear: Callable[..., torch.Tensor]   # linear(a [M, K], w [N, K], out_dtype=None) -> [M, N]
    kernel_libraries: tuple[str, ...] = ()  # what `linear` itself needs compiled
    extras: dict = field(default_factory=dict)


class Part:
    def __init__(self, params: dict, prefix: str):
        self.params = dict(params)
        self.prefix = prefix

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime

    def parts(self) -> list["Part"]:
        """The parts this one is made of (a block's norms, mixer and feed-forward; a mixer's
        position encoding), so that a model can ask all of them what they need."""
        return []

    def kernel_libraries(self, dtype: torch.dtype) -> tuple[str, ...]:
        """Names of the kernel libraries this part launches in a run of `dtype`: the package's own
        (`csrc/build.py`'s SOURCES) or sources registered with `csrc.build.register_source`. They are
        compiled before the model's first step."""
        return ()

    def tile_sizes(self, dtype: torch.dtype) -> tuple[int, ...]:
        """Query-tile sizes whose (sequence, first query) lists every step's batch must carry."""
        return ()

    def require(self, *names: str) -> None:
        missing = [n for n in names if n not in self.params]
        if missing:
            raise ValueError(f"{type(self).__name__} lacks parameters {missing}")


def walk_parts(part: "Part"):
    """`part` and everything below it, depth first."""
    yield part
    for child in part.parts():
        if child is not None:
            yield from walk_parts(child)


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
