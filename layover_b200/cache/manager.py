"""The cache manager: pages of keys and values with a block table per request, and slots of
fixed-size state per request.

The model's mixers say what they need (`PagedKVNeed`, `StateNeed`). Schedule entries with the
same need form a *group*: a group of paged needs owns one pool tensor
`[layers of the group, 2 (K, V), pages + 1, kv_heads, page_tokens, head_dim]` and one page
allocator, and every request has one block table per group. (The reference has a single pool
for its one kind of layer, layover/kv/paged_cache.py:26-49, laid out block-major for its swap
path; here a page of one head is a contiguous run of page_tokens * head_dim elements per
layer, which is what the attention kernels read.) The last page of each pool is a scratch page
that is never handed out: padded rows of a captured decode step and table entries whose page
was given back point at it.

A group with a window only keeps the pages that a later query can still see: after a step,
pages that lie wholly below `tokens - window + 1` go back to the free list and are reused.
State groups own `[slots + 1, *shape]`; a request's slot is zeroed when it is opened.

Beside the mixers' state every request has one *record* of `record_words` int32 words on the
device, `records[slot]`, written whole when the request is opened and never touched by the host
again: kernels index it by the request's slot, so a captured CUDA graph sees a fixed address.
What the words mean is the business of whoever writes and reads them (the sampler keeps the
request's seed, counter, temperature and last token there); the manager only hands out the row.
(The reference keeps such facts on the host, layover/engine.py:39-40; its nearest device-side
relative is the packed row at a fixed address of layover/decode_graphs.py:56-77.)

All bookkeeping is on the host and works without a device (`device=None` allocates no pools),
which is how the scheduler and the property tests use it.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import PagedKVNeed, StateNeed
from .allocator import BlockAllocator, OutOfBlocks


@dataclass
class PagedGroup:
    need: PagedKVNeed
    entries: list[int]                 # schedule entries that write into this group, in layer order
    allocator: BlockAllocator
    pool: torch.Tensor | None = None   # [layers, 2, pages + 1, kv_heads, page_tokens, head_dim]

    @property
    def scratch_page(self) -> int:
        return self.allocator.num_blocks


@dataclass
class StateGroup:
    need: StateNeed
    entries: list[int]
    pool: torch.Tensor | None = None   # [entries, slots + 1, *shape]


@dataclass
class CacheView:
    """What one schedule entry's mixer sees of the cache."""
    kind: str                          # "paged" or "state"
    group: int                         # index among the groups of its kind
    layer: int                         # index inside the group's pool
    writes: bool = True                # False when the entry reads another entry's keys and values
    k_pool: torch.Tensor | None = None # [pages + 1, kv_heads, page_tokens, head_dim]
    v_pool: torch.Tensor | None = None
    pool: torch.Tensor | None = None   # the group's whole pool [layers, 2, pages + 1, kv_heads, page_tokens, head_dim]
    state: torch.Tensor | None = None  # [slots + 1, *shape]
    page_tokens: int = 0
    need: object = None


@dataclass
class BlockTable:
    """One request's pages in one group; `first_live` pages at the front were given back."""
    blocks: list[int] = field(default_factory=list)
    first_live: int = 0


@dataclass
class SequenceCache:
    """Everything the cache holds for one live request."""
    request_id: str
    slot: int
    tables: list[BlockTable]
    num_tokens: int = 0
    closed: bool = False


class CacheManager:
    def __init__(self, needs: list[tuple[int, object, int | None]], num_blocks: int, block_tokens: int = 16,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | str | None = None,
                 max_requests: int = 64, record_words: int = 8):
        """`needs`: for every schedule entry (entry index, its need or None, the entry whose cache
        it reads instead of its own or None). `num_blocks` pages per paged group."""
        if block_tokens <= 0:
            raise ValueError("block_tokens must be positive")
        self.block_tokens = block_tokens
        self.dtype = dtype
        self.device = None if device is None else torch.device(device)
        self.max_requests = max_requests
        self.paged: list[PagedGroup] = []
        self.states: list[StateGroup] = []
        self.views: dict[int, CacheView] = {}
        own = {entry: need for entry, need, reads in needs if reads is None and need is not None}
        for entry, need in own.items():
            if isinstance(need, PagedKVNeed):
                group = next((g for g in self.paged if g.need == need), None)
                if group is None:
                    group = PagedGroup(need, [], BlockAllocator(num_blocks))
                    self.paged.append(group)
                group.entries.append(entry)
                self.views[entry] = CacheView("paged", self.paged.index(group), len(group.entries) - 1,
                                              page_tokens=block_tokens, need=need)
            elif isinstance(need, StateNeed):
                group = next((g for g in self.states if g.need == need), None)
                if group is None:
                    group = StateGroup(need, [])
                    self.states.append(group)
                group.entries.append(entry)
                self.views[entry] = CacheView("state", self.states.index(group), len(group.entries) - 1, need=need)
            else:
                raise TypeError(f"schedule entry {entry}: unknown cache need {need!r}")
        for entry, need, reads in needs:
            if reads is not None:
                if reads not in self.views or self.views[reads].kind != "paged":
                    raise ValueError(f"schedule entry {entry} reads the cache of entry {reads}, which has no pages")
                src = self.views[reads]
                self.views[entry] = CacheView("paged", src.group, src.layer, writes=False,
                                              page_tokens=block_tokens, need=src.need)
        self._slots = BlockAllocator(max_requests)
        self.live: dict[str, SequenceCache] = {}
        self.record_words = int(record_words)
        self.records: torch.Tensor | None = None     # [max_requests + 1, record_words] int32 on the device
        self._record_staging = None                  # the same rows in pinned host memory, and when each was last sent
        self._record_sent: list = [None] * (max_requests + 1)
        if self.device is not None:
            self._allocate_pools()

    # ------------------------------------------------------------------ device memory
    def _allocate_pools(self) -> None:
        for group in self.paged:
            need = group.need
            group.pool = torch.zeros(
                (len(group.entries), 2, group.allocator.num_blocks + 1, need.kv_heads, self.block_tokens, need.head_dim),
                dtype=self.dtype, device=self.device)
        for group in self.states:
            group.pool = torch.zeros((len(group.entries), self.max_requests + 1, *group.need.shape),
                                     dtype=group.need.dtype, device=self.device)
        self.records = torch.zeros((self.max_requests + 1, self.record_words), dtype=torch.int32, device=self.device)
        if self.device.type == "cuda":
            self._record_staging = torch.zeros((self.max_requests + 1, self.record_words), dtype=torch.int32,
                                               pin_memory=True)
        for view in self.views.values():
            if view.kind == "paged":
                pool = self.paged[view.group].pool
                view.k_pool, view.v_pool, view.pool = pool[view.layer, 0], pool[view.layer, 1], pool
            else:
                view.state = self.states[view.group].pool[view.layer]

    def view(self, entry: int) -> CacheView | None:
        return self.views.get(entry)

    @property
    def scratch_slot(self) -> int:
        return self.max_requests

    @property
    def num_free_slots(self) -> int:
        return self._slots.num_free

    def pool_bytes(self) -> int:
        pools = [g.pool for g in self.paged] + [g.pool for g in self.states] + [self.records]
        return sum(p.numel() * p.element_size() for p in pools if p is not None)

    # ------------------------------------------------------------------ arithmetic
    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.block_tokens)

    @property
    def num_blocks(self) -> int:
        return min((g.allocator.num_blocks for g in self.paged), default=0)

    @property
    def num_free(self) -> int:
        return min((g.allocator.num_free for g in self.paged), default=0)

    def _first_needed_page(self, group: PagedGroup, first_query: int) -> int:
        """Pages below this index hold no key that a query at `first_query` or later can see."""
        if group.need.window is None:
            return 0
        return max(0, first_query - group.need.window + 1) // self.block_tokens

    def peak_blocks(self, group_index: int, total_tokens: int, chunk: int) -> int:
        """The most pages of a group that a request of `total_tokens` holds at any time when it is
        fed at most `chunk` tokens a step."""
        group = self.paged[group_index]
        if group.need.window is None:
            return self.blocks_for(total_tokens)
        span = min(total_tokens, group.need.window - 1 + max(1, chunk))
        return min(self.blocks_for(total_tokens), span // self.block_tokens + 2)

    def blocks_missing(self, seq: SequenceCache, new_total: int) -> list[int]:
        """Per paged group: pages to allocate before tokens [seq.num_tokens, new_total) can be written."""
        out = []
        for group, table in zip(self.paged, seq.tables):
            first = max(len(table.blocks), self._first_needed_page(group, seq.num_tokens))
            out.append(max(0, self.blocks_for(new_total) - first))
        return out

    # ------------------------------------------------------------------ life of a request
    def open(self, request_id: str, record: list[int] | None = None) -> SequenceCache:
        """A slot and empty tables for a new request. `record` (up to `record_words` int32 values, the
        rest zero) becomes the request's record on the device; the mixers' state of the slot is zeroed."""
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already open")
        if record is not None and len(record) > self.record_words:
            raise ValueError(f"a record holds {self.record_words} words, got {len(record)}")
        try:
            slot = self._slots.alloc(1)[0]
        except OutOfBlocks:
            raise OutOfBlocks(f"all {self.max_requests} request slots are in use") from None
        for group in self.states:
            if group.pool is not None:
                group.pool[:, slot].zero_()
        if self.records is not None:
            words = torch.zeros(self.record_words, dtype=torch.int32)
            if record:
                words[: len(record)] = torch.tensor(record, dtype=torch.int64).to(torch.int32)
            if self._record_staging is not None:
                # stream-ordered behind every kernel that still uses the slot's previous owner
                if self._record_sent[slot] is not None:
                    self._record_sent[slot].synchronize()
                self._record_staging[slot] = words
                self.records[slot].copy_(self._record_staging[slot], non_blocking=True)
                self._record_sent[slot] = torch.cuda.Event()
                self._record_sent[slot].record()
            else:
                self.records[slot] = words
        seq = SequenceCache(request_id, slot, [BlockTable() for _ in self.paged])
        self.live[request_id] = seq
        return seq

    def grow(self, seq: SequenceCache, new_total: int) -> None:
        """Make room for tokens up to `new_total`, in every group or in none (OutOfBlocks)."""
        if seq.closed:
            raise ValueError(f"request {seq.request_id!r} is closed")
        missing = self.blocks_missing(seq, new_total)
        for group, count in zip(self.paged, missing):
            if count > group.allocator.num_free:
                raise OutOfBlocks(f"need {count} blocks, {group.allocator.num_free} free")
        for group, table in zip(self.paged, seq.tables):
            first_needed = self._first_needed_page(group, seq.num_tokens)
            for index in range(len(table.blocks), self.blocks_for(new_total)):
                if index < first_needed:  # a page no query of this or a later step can see
                    table.blocks.append(group.scratch_page)
                    table.first_live = max(table.first_live, index + 1)
                else:
                    table.blocks.append(group.allocator.alloc(1)[0])

    def commit(self, seq: SequenceCache, new_total: int) -> None:
        """The step that wrote tokens up to `new_total` has been issued: count them and give back
        the pages that a window has passed."""
        if new_total < seq.num_tokens:
            raise ValueError("a request's token count cannot shrink")
        if any(self.blocks_for(new_total) > len(t.blocks) for t in seq.tables):
            raise ValueError("commit past the pages that grow() made")
        seq.num_tokens = new_total
        for group, table in zip(self.paged, seq.tables):
            first_needed = min(self._first_needed_page(group, new_total), len(table.blocks))
            for index in range(table.first_live, first_needed):
                if table.blocks[index] != group.scratch_page:
                    group.allocator.free(table.blocks[index])
                    table.blocks[index] = group.scratch_page
            table.first_live = max(table.first_live, first_needed)

    def close(self, seq: SequenceCache) -> None:
        """Give back every page and the state slot."""
        if seq.closed:
            raise ValueError(f"request {seq.request_id!r} was closed before")
        for group, table in zip(self.paged, seq.tables):
            for block in table.blocks:
                if block != group.scratch_page:
                    group.allocator.free(block)
            table.blocks = []
            table.first_live = 0
        self._slots.free(seq.slot)
        seq.closed = True
        seq.num_tokens = 0
        del self.live[seq.request_id]

    release = close

    # ------------------------------------------------------------------ checks
    def check_tables(self, seq: SequenceCache, tokens: int | None = None) -> None:
        """What a kernel cannot check for itself, before every launch (layover/kv/paged_cache.py:160-165):
        the request is the one this manager opened, its slot is inside the pool, every page id of
        its tables is inside its group's pool and held (or the scratch page), and the tables cover
        `tokens` tokens (default: those it holds)."""
        if self.live.get(seq.request_id) is not seq:
            raise ValueError(f"request {seq.request_id!r} is not open in this cache")
        if not 0 <= seq.slot < self.max_requests or len(seq.tables) != len(self.paged):
            raise ValueError(f"request {seq.request_id!r}: slot {seq.slot} or its tables do not belong to this cache")
        needed = self.blocks_for(seq.num_tokens if tokens is None else tokens)
        for group, table in zip(self.paged, seq.tables):
            if len(table.blocks) < needed:
                raise ValueError(f"request {seq.request_id!r}: {needed} pages needed, its table has {len(table.blocks)}")
            held = group.allocator.is_held
            for block in table.blocks:
                if block != group.scratch_page and not held(block):
                    raise ValueError(f"request {seq.request_id!r}: block {block} is not an allocated page of its pool")

    def check_row(self, group_index: int, row, request_id: str = "?") -> None:
        """The same check on one request's page ids as an int32 numpy array (what the batch builder
        is about to send to the device): every id is the scratch page or a held page of the group's
        pool. Vectorised, so that it costs little on every step."""
        import numpy as np

        group = self.paged[group_index]
        if row.size == 0:
            return
        low, high = int(row.min()), int(row.max())
        if low < 0 or high > group.scratch_page:
            raise ValueError(f"request {request_id!r}: page id {low if low < 0 else high} is outside its pool of "
                             f"{group.allocator.num_blocks} pages")
        real = row[row != group.scratch_page]
        if real.size and not np.frombuffer(group.allocator._out, dtype=np.uint8)[real].all():
            bad = int(real[np.frombuffer(group.allocator._out, dtype=np.uint8)[real] == 0][0])
            raise ValueError(f"request {request_id!r}: block {bad} is not an allocated page of its pool")

    def check(self) -> None:
        """No page lost, held twice or both free and held, over all live requests."""
        for index, group in enumerate(self.paged):
            group.allocator.check()
            held = [b for seq in self.live.values() for b in seq.tables[index].blocks if b != group.scratch_page]
            if len(held) != len(set(held)):
                raise AssertionError("a page is held by two tables")
            if len(held) != group.allocator.num_used:
                raise AssertionError(f"{group.allocator.num_used} pages are out, {len(held)} are in tables")
            for block in held:
                if not group.allocator.is_held(block):
                    raise AssertionError(f"page {block} is in a table and on the free list")
        self._slots.check()
        if self._slots.num_used != len(self.live):
            raise AssertionError("state slots and live requests disagree")
