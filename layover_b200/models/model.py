"""A model built from a `ModelSpec`: embedding, scheduled blocks, final norm, output matrix.

`Model.forward(batch, cache)` is the device side of a step: it runs exactly the tokens of the
batch, reads and writes the cache through the views the cache manager made for each schedule
entry, and returns 32-bit logits for the wanted rows only (layover/model.py:199-255 keep two
functions, one per kind of step; here one serves every mix). It reads nothing back to the host.
"""

from __future__ import annotations

import torch

from .. import ops
from .. import profiling
from ..parts.base import Runtime, build_part, walk_parts
from ..weights.loader import TensorSpec
from .spec import ModelSpec


class Model:
    def __init__(self, spec: ModelSpec, config=None):
        self.spec = spec
        self.cfg = config
        self.blocks = [build_part("block", layer.block, layer.prefix) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, spec.norm_prefix)
        self.embedding = self.head = None
        self.runtime: Runtime | None = None
        self._range_names = [f"layer{e.layer}" for e in spec.schedule]

    # ---- weights
    def tensor_specs(self) -> list[TensorSpec]:
        s = self.spec
        specs = [TensorSpec(s.embedding, (s.vocab_size, s.hidden_size))]
        for block in self.blocks:
            specs += block.tensor_specs()
        specs += self.final_norm.tensor_specs()
        if s.head is not None:
            specs.append(TensorSpec(s.head, (s.vocab_size, s.hidden_size)))
        return specs

    def bind(self, tensors: dict[str, torch.Tensor], runtime: Runtime) -> "Model":
        self.runtime = runtime
        self.embedding = tensors[self.spec.embedding]
        self.head = self.embedding if self.spec.head is None else tensors[self.spec.head]
        for block in self.blocks:
            block.bind(tensors, runtime)
        self.final_norm.bind(tensors, runtime)
        return self

    @property
    def dtype(self) -> torch.dtype:
        return self.runtime.dtype

    @property
    def device(self) -> torch.device:
        return self.runtime.device

    def weight_bytes(self) -> int:
        """Bytes of every weight tensor a decode step reads once (the embedding counts only as the head)."""
        seen, total = set(), 0
        for block in self.blocks:
            for part in walk_parts(block):
                for value in vars(part).values():
                    if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                        seen.add(value.data_ptr())
                        total += value.numel() * value.element_size()
        total += self.head.numel() * self.head.element_size()
        return total

    # ---- cache
    def cache_needs(self) -> list[tuple[int, object, int | None]]:
        """(schedule entry, its need, the entry whose cache it reads) for the cache manager."""
        return [(index, self.blocks[entry.layer].cache_need(), entry.reads_cache_of)
                for index, entry in enumerate(self.spec.schedule)]

    def all_parts(self):
        """Every part of the model, the blocks' sub-parts included."""
        for top in [*self.blocks, self.final_norm]:
            yield from walk_parts(top)

    def kernel_libraries(self, dtype: torch.dtype, runtime: Runtime | None = None) -> tuple[str, ...]:
        """What has to be compiled before the first step of a run of `dtype`: the model's own kernels
        (embedding, sampling), the run's matrix product and whatever the parts say they launch."""
        runtime = runtime or self.runtime
        names = ["elementwise", "sampling", *(runtime.kernel_libraries if runtime else ())]
        for part in self.all_parts():
            names += part.kernel_libraries(dtype)
        return tuple(dict.fromkeys(names))

    def tile_sizes(self) -> tuple[int, ...]:
        """Query-tile sizes that the parts want listed in every batch."""
        sizes = [size for part in self.all_parts() for size in part.tile_sizes(self.runtime.dtype)]
        return tuple(sorted(set(sizes)))

    # ---- one step
    def forward(self, batch, cache) -> torch.Tensor:
        rt = self.runtime
        batch.shared.clear()    # what parts share within a step (rotary tables) is made anew by every run
        x = torch.empty((batch.n_tokens, self.spec.hidden_size), dtype=rt.dtype, device=rt.device)
        records = getattr(cache, "records", None)      # tokens the host has not seen yet come from the requests' records
        ops.embed(batch.token_ids, self.embedding, x, batch.token_src if records is not None else None, records)
        delta = None
        if profiling.active():
            for index, entry in enumerate(self.spec.schedule):
                with profiling.nvtx_range(self._range_names[index]):
                    x, delta = self.blocks[entry.layer].forward(x, delta, batch, cache.view(index))
        else:
            for index, entry in enumerate(self.spec.schedule):
                x, delta = self.blocks[entry.layer].forward(x, delta, batch, cache.view(index))
        if batch.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        h = self.final_norm.forward(x, delta, rows=batch.logit_rows)
        return rt.linear(h, self.head, out_dtype=torch.float32)


def assemble(spec: ModelSpec, config=None) -> Model:
    return Model(spec, config)
