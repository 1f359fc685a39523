"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

`StepFunction(model, cache)(entries)` makes room in the cache for every entry's tokens (all
entries or none: `OutOfBlocks` leaves the cache as it was), packs the batch with one copy to the
device, runs the model over exactly those tokens and counts them into the requests. Portions of
prompts and single decoded tokens share a batch, cut anywhere. The reference runs one call per
prefilling request and then one decode batch (layover/engine.py:156-189); here both are one
batch.

A step of single tokens only (every live request decoding) can replay a captured CUDA graph:
one graph per batch size bucket, with the batch's descriptors at a fixed address and unused rows
padded onto the scratch page (the reference captures batch 1, 2, 4, 8 the same way,
layover/decode_graphs.py:25-100).
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..profiling import nvtx_range
from .batch import BatchBuilder, BatchCapacity, StepEntry

DEFAULT_GRAPH_SIZES = (1, 2, 4, 8, 16, 32, 64)


class _DecodeGraph:
    def __init__(self, size: int, step: "StepFunction"):
        self.size = size
        cache = step.cache
        self.capacity = BatchCapacity(size, step.graph_table_width)
        words = BatchBuilder.buffer_size(self.capacity, len(cache.paged), step.builder.tile_sizes)
        self.buffer = torch.zeros(words, dtype=torch.int32, device=step.device)
        self.graph = None
        self.logits = None

    def capture(self, step: "StepFunction", pool):
        batch = step.builder.build([], self.capacity, self.buffer)   # padding rows only
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step.model.forward(batch, step.cache)
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        with torch.cuda.graph(self.graph, pool=pool):
            self.logits = step.model.forward(batch, step.cache)
        self.launches = ops.LAUNCHES - before      # kernels one replay runs
        return self.graph.pool()


class StepFunction:
    def __init__(self, model, cache: CacheManager, cuda_graphs: bool = False,
                 graph_sizes: tuple[int, ...] = DEFAULT_GRAPH_SIZES, graph_max_tokens: int | None = None):
        self.model, self.cache = model, cache
        self.device = model.device
        self.builder = BatchBuilder(cache, self.device, model.tile_sizes())
        self.vocab_size = model.spec.vocab_size
        self.max_position = model.spec.max_position
        self.cuda_graphs = cuda_graphs
        self.graph_sizes = tuple(sorted(s for s in graph_sizes if s <= cache.max_requests))
        limit = graph_max_tokens or self.max_position
        self.graph_table_width = max(1, min(cache.blocks_for(limit), max(cache.num_blocks, 1)))
        self._graphs: dict[int, _DecodeGraph] = {}
        self._graph_pool = None
        self.steps = 0
        self.graph_replays = 0
        self.replayed_launches = 0

    # ---- checks the kernels cannot make
    def _check(self, entries: list[StepEntry], previous_rows: int = 0) -> None:
        seen = set()
        for entry in entries:
            seq = entry.seq
            if seq.closed:
                raise ValueError(f"request {seq.request_id!r} is closed")
            if id(seq) in seen:
                raise ValueError(f"request {seq.request_id!r} appears twice in one step")
            seen.add(id(seq))
            if not entry.tokens:
                raise ValueError(f"request {seq.request_id!r}: no tokens in this step")
            if seq.num_tokens + len(entry.tokens) > self.max_position:
                raise ValueError(f"request {seq.request_id!r} would exceed {self.max_position} positions")
            for token in entry.tokens:
                if not -previous_rows <= token < self.vocab_size:
                    raise ValueError(f"request {seq.request_id!r}: token {token} is outside the vocabulary")

    def _reserve(self, entries: list[StepEntry]) -> None:
        """Pages for every entry or for none."""
        cache = self.cache
        totals = [0] * len(cache.paged)
        for entry in entries:
            for g, count in enumerate(cache.blocks_missing(entry.seq, entry.seq.num_tokens + len(entry.tokens))):
                totals[g] += count
        for group, need in zip(cache.paged, totals):
            if need > group.allocator.num_free:
                from ..cache.allocator import OutOfBlocks
                raise OutOfBlocks(f"this step needs {need} blocks, {group.allocator.num_free} free")
        for entry in entries:
            cache.grow(entry.seq, entry.seq.num_tokens + len(entry.tokens))

    # ---- the step
    def __call__(self, entries: list[StepEntry], previous_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Logits [wanted rows, vocab] in 32-bit on the device, in the order of entries and want.

        `previous_tokens` (int32, on the device) are the tokens the step before sampled; entries name
        them with negative token values, so a step can be launched before the host has read them.
        After a replayed graph the result is a view of the graph's output, which the next replay
        of the same bucket overwrites: use it (sample, copy) before the next step."""
        self._check(entries, 0 if previous_tokens is None else previous_tokens.shape[0])
        self._reserve(entries)
        with nvtx_range("step"):
            graph = self._graph_for(entries)
            if graph is not None:
                batch = self.builder.build(entries, graph.capacity, graph.buffer)
                if batch.device_tokens:
                    ops.patch_tokens(batch.token_ids, batch.token_src, previous_tokens)
                graph.graph.replay()
                self.graph_replays += 1
                self.replayed_launches += graph.launches
                rows = [i for i, e in enumerate(entries) if e.want]
                logits = graph.logits[: len(entries)] if len(rows) == len(entries) else graph.logits[rows]
            else:
                batch = self.builder.build(entries)
                if batch.device_tokens:
                    ops.patch_tokens(batch.token_ids, batch.token_src, previous_tokens)
                logits = self.model.forward(batch, self.cache)
        for entry in entries:
            self.cache.commit(entry.seq, entry.seq.num_tokens + len(entry.tokens))
        self.steps += 1
        return logits

    def _graph_for(self, entries: list[StepEntry]) -> _DecodeGraph | None:
        if not self.cuda_graphs or any(len(e.tokens) != 1 or e.want not in ([0], []) for e in entries):
            return None
        size = next((s for s in self.graph_sizes if s >= len(entries)), None)
        if size is None:
            return None
        if max(self.cache.blocks_for(e.seq.num_tokens + 1) for e in entries) > self.graph_table_width:
            return None
        graph = self._graphs.get(size)
        if graph is None:
            graph = self._capture(size)
        return graph

    def _capture(self, size: int) -> _DecodeGraph:
        graph = _DecodeGraph(size, self)
        self._graph_pool = graph.capture(self, self._graph_pool)
        self._graphs[size] = graph
        return graph

    def capture_all(self) -> None:
        """Capture every bucket now, largest first so that the smaller ones fit in its memory pool."""
        for size in reversed(self.graph_sizes):
            if size not in self._graphs:
                self._capture(size)
