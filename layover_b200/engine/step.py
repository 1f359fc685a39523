"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

`StepFunction(model, cache)(entries)` makes room in the cache for every entry's tokens (all
entries or none: `OutOfBlocks` leaves the cache as it was), packs the batch with one copy to the
device, runs the model over exactly those tokens and counts them into the requests. Portions of
prompts and single decoded tokens share a batch, cut anywhere. The reference runs one call per
prefilling request and then one decode batch (layover/engine.py:156-189); here both are one
batch. `sample(entries)` does the same and then chooses a token for every wanted row on the
device (`sampling.Sampler`), returning them on their way to the host.

A step of single tokens only (every live request decoding) can replay a captured CUDA graph: one
graph per (batch size bucket, block-table width bucket, requests about equally long or not: the
decode attention plans its launch differently for the two), with the batch's descriptors at a fixed
address and unused rows padded onto the scratch page and the scratch record (the reference
captures batch 1, 2, 4, 8 the same way, layover/decode_graphs.py:25-100). The width bucket is the
request's pages rounded up to a power of two, so the attention's split count is planned for about
the context that is really there, not for the longest a request could ever get.

A step that is one prompt portion of a size named in `portion_graph_tokens` (the scheduler's
prefill chunk) replays a graph too, one per (size, width bucket, last token's logits wanted or
not): a portion is a few hundred launches, and the first short ones (embedding, norms, rotation)
otherwise wait for the host between them.
"""

from __future__ import annotations

import torch

from .. import ops, profiling
from ..cache.allocator import OutOfBlocks
from ..cache.manager import CacheManager
from ..sampling.sampler import PendingTokens, Sampler
from .batch import DEVICE_TOKEN, BatchBuilder, BatchCapacity, StepEntry

DEFAULT_GRAPH_SIZES = (1, 2, 4, 8, 16, 32, 64)
MIN_GRAPH_WIDTH = 64          # pages: the smallest block-table bucket a graph is captured for


class _CapturedStep:
    """One captured step of fixed sizes (`capacity`), with or without sampling of its logit rows."""

    def __init__(self, capacity: BatchCapacity, sampled: bool, step: "StepFunction", plan_ctx: tuple[int, int] | None = None):
        self.capacity, self.sampled = capacity, sampled
        self.plan_ctx = plan_ctx      # (longest, mean) context that the decode attention of this graph is planned for
        self.size = (1 if capacity.want_last else 0) if capacity.portion else capacity.seqs   # logit rows
        cache = step.cache
        words = BatchBuilder.buffer_size(self.capacity, len(cache.paged), step.builder.tile_sizes)
        self.buffer = torch.zeros(words, dtype=torch.int32, device=step.device)
        self.tokens = None
        if sampled:
            self.tokens = torch.zeros(self.size + step.sampler.n_status, dtype=torch.int32, device=step.device)
        self.graph = None
        self.logits = None
        self.launches = 0

    def _run(self, step: "StepFunction", batch):
        logits = step.model.forward(batch, step.cache)
        if self.sampled:
            step.sampler.sample_into(logits, batch, self.tokens)
        return logits

    def capture(self, step: "StepFunction", pool):
        batch = step.builder.build([], self.capacity, self.buffer, self.plan_ctx)   # padding rows only
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._run(step, batch)
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        with torch.cuda.graph(self.graph, pool=pool):
            self.logits = self._run(step, batch)
        self.launches = ops.LAUNCHES - before      # kernels one replay runs
        return self.graph.pool()


class StepFunction:
    def __init__(self, model, cache: CacheManager, cuda_graphs: bool = False,
                 graph_sizes: tuple[int, ...] = DEFAULT_GRAPH_SIZES, graph_max_tokens: int | None = None,
                 sampler: Sampler | None = None, portion_graph_tokens: tuple[int, ...] = ()):
        self.model, self.cache = model, cache
        self.device = model.device
        self.builder = BatchBuilder(cache, self.device, model.tile_sizes())
        self.vocab_size = model.spec.vocab_size
        self.max_position = model.spec.max_position
        self.cuda_graphs = cuda_graphs
        # False: a step that has a graph runs the graph's own fixed-size batch through the kernels
        # launch by launch instead of replaying it (the same launches with the same arguments; what
        # a replay must reproduce bit for bit, which tests and the benchmark check)
        self.replay_graphs = True
        self.graph_sizes = tuple(sorted(s for s in graph_sizes if s <= cache.max_requests))
        self.portion_graph_tokens = tuple(portion_graph_tokens)   # sizes of lone prompt portions to capture
        limit = graph_max_tokens or self.max_position
        self.graph_table_width = max(1, min(cache.blocks_for(limit), max(cache.num_blocks, 1)))
        if sampler is None:
            sampler = Sampler(self.device, cache.records, model.kernel_libraries(model.dtype))
        self.sampler = sampler
        self._graphs: dict[tuple, _CapturedStep] = {}
        self._graph_pool = None
        self.steps = 0
        self.graph_replays = 0
        self.replayed_launches = 0

    # ---- checks the kernels cannot make
    def _check(self, entries: list[StepEntry]) -> None:
        seen = set()
        live = self.cache.live
        for entry in entries:
            seq = entry.seq
            if seq.closed or live.get(seq.request_id) is not seq:
                raise ValueError(f"request {seq.request_id!r} is closed or does not belong to this cache")
            if id(seq) in seen:
                raise ValueError(f"request {seq.request_id!r} appears twice in one step")
            seen.add(id(seq))
            if not entry.tokens:
                raise ValueError(f"request {seq.request_id!r}: no tokens in this step")
            if not 0 <= seq.slot < self.cache.max_requests:
                raise ValueError(f"request {seq.request_id!r}: state slot {seq.slot} is outside the cache")
            if seq.num_tokens + len(entry.tokens) > self.max_position:
                raise ValueError(f"request {seq.request_id!r} would exceed {self.max_position} positions")
            low, high = min(entry.tokens), max(entry.tokens)
            if low == DEVICE_TOKEN and len(entry.tokens) == 1:
                continue
            if low == DEVICE_TOKEN:
                raise ValueError(f"request {seq.request_id!r}: a token still on the device comes alone")
            if low < 0 or high >= self.vocab_size:
                raise ValueError(f"request {seq.request_id!r}: token {low if low < 0 else high} is outside the vocabulary")

    def _reserve(self, entries: list[StepEntry]) -> None:
        """Pages for every entry or for none."""
        cache = self.cache
        totals = [0] * len(cache.paged)
        for entry in entries:
            for g, count in enumerate(cache.blocks_missing(entry.seq, entry.seq.num_tokens + len(entry.tokens))):
                totals[g] += count
        for group, need in zip(cache.paged, totals):
            if need > group.allocator.num_free:
                raise OutOfBlocks(f"this step needs {need} blocks, {group.allocator.num_free} free")
        for entry in entries:
            cache.grow(entry.seq, entry.seq.num_tokens + len(entry.tokens))

    # ---- the step
    def __call__(self, entries: list[StepEntry]) -> torch.Tensor:
        """Logits [wanted rows, vocab] in 32-bit on the device, in the order of entries and want.

        After a replayed graph the result is a view of the graph's output, which the next replay
        of the same graph overwrites: use it (copy it) before the next step."""
        return self._step(entries, sampled=False)

    def sample(self, entries: list[StepEntry]) -> PendingTokens:
        """The same step, then one token for every wanted row, chosen on the device as the requests'
        records say; `result()` of what is returned waits for them (in the order of entries and want)."""
        return self._step(entries, sampled=True)

    def _step(self, entries: list[StepEntry], sampled: bool):
        self._check(entries)
        self._reserve(entries)
        with profiling.nvtx_range("step"):
            graph = self._graph_for(entries, sampled)
            if graph is not None:
                batch = self.builder.build(entries, graph.capacity, graph.buffer, graph.plan_ctx)
                if self.replay_graphs:
                    graph.graph.replay()
                    logits = graph.logits
                    self.graph_replays += 1
                    self.replayed_launches += graph.launches
                else:
                    logits = graph._run(self, batch)
                rows = [i for i, e in enumerate(entries) if e.want]
                if sampled and graph.size == 0:
                    out = PendingTokens(None, None, 0, 0, self.sampler)
                elif sampled:
                    if len(rows) != len(entries):
                        raise ValueError("a replayed sampled step samples every row")     # _graph_for saw to it
                    out = self.sampler.collect(graph.tokens, len(entries), graph.size)
                else:
                    out = logits[: len(entries)] if len(rows) == len(entries) else logits[rows]
            else:
                batch = self.builder.build(entries)
                out = self.model.forward(batch, self.cache)
                if sampled:
                    out = self.sampler.launch(out, batch)
        for entry in entries:
            self.cache.commit(entry.seq, entry.seq.num_tokens + len(entry.tokens))
        self.steps += 1
        return out

    def graph_width_for(self, pages: int) -> int | None:
        """The block-table bucket for a longest request of `pages` pages; None: wider than any graph."""
        if pages > self.graph_table_width:
            return None
        width = MIN_GRAPH_WIDTH
        while width < pages:
            width *= 2
        return min(width, self.graph_table_width)

    def _graph_for(self, entries: list[StepEntry], sampled: bool) -> _CapturedStep | None:
        if not self.cuda_graphs:
            return None
        if len(entries) == 1 and len(entries[0].tokens) in self.portion_graph_tokens and len(entries[0].tokens) > 1:
            return self._portion_graph_for(entries[0], sampled)
        if any(len(e.tokens) != 1 for e in entries):
            return None
        if any(e.want != [0] for e in entries) if sampled else any(e.want not in ([0], []) for e in entries):
            return None
        size = next((s for s in self.graph_sizes if s >= len(entries)), None)
        if size is None:
            return None
        lengths = [e.seq.num_tokens + 1 for e in entries]
        width = self.graph_width_for(self.cache.blocks_for(max(lengths)))
        if width is None:
            return None
        skew = 2 if 2 * max(lengths) * len(lengths) > 3 * sum(lengths) else 1     # the longest is 1.5 times the mean or more
        graph = self._graphs.get((size, width, sampled, skew))
        if graph is None:
            graph = self._capture(size, width, sampled, skew)
        return graph

    def _portion_graph_for(self, entry: StepEntry, sampled: bool) -> _CapturedStep | None:
        count = len(entry.tokens)
        if entry.want not in ([], [count - 1]):
            return None
        width = self.graph_width_for(self.cache.blocks_for(entry.seq.num_tokens + count))
        if width is None:
            return None
        want_last = bool(entry.want)
        key = ("portion", count, width, want_last, sampled and want_last)
        graph = self._graphs.get(key)
        if graph is None:
            graph = _CapturedStep(BatchCapacity(1, width, count, want_last), sampled and want_last, self)
            self._graph_pool = graph.capture(self, self._graph_pool)
            self._graphs[key] = graph
        return graph

    def _capture(self, size: int, width: int, sampled: bool, skew: int = 1) -> _CapturedStep:
        """`skew` 1: a step whose requests are about equally long; 2: one whose longest request has 1.5
        times the mean or more (the decode attention cuts the contexts further for those)."""
        longest = width * self.cache.block_tokens
        graph = _CapturedStep(BatchCapacity(size, width), sampled, self, (longest, longest // skew))
        self._graph_pool = graph.capture(self, self._graph_pool)
        self._graphs[(size, width, sampled, skew)] = graph
        return graph

    def capture_all(self, tokens: int | None = None, sampled: bool = True, from_tokens: int | None = None,
                    skews: tuple[int, ...] = (1,)) -> None:
        """Capture now, instead of at first use, every batch-size bucket for requests that hold between
        `from_tokens` (default: `tokens`) and `tokens` tokens (default: the widest table): every
        block-table bucket in that range, largest first so that the smaller ones fit in its memory pool.
        `skews`: the classes of steps to capture (1: requests about equally long; 2: the longest has 1.5
        times the mean or more); a class that is not captured here is captured when a step first needs it."""
        top = self.graph_width_for(self.cache.blocks_for(tokens)) if tokens else self.graph_table_width
        if top is None:
            raise ValueError(f"{tokens} tokens are more than a captured step can hold")
        low = self.graph_width_for(self.cache.blocks_for(from_tokens)) if from_tokens else top
        widths = sorted({w for w in (self.graph_width_for(p) for p in range(low, top + 1)) if w is not None}, reverse=True)
        for width in widths:
            for size in reversed(self.graph_sizes):
                for skew in skews:
                    if (size, width, sampled, skew) not in self._graphs:
                        self._capture(size, width, sampled, skew)
