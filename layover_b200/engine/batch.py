"""One step's batch as the kernels see it: flat token arrays and per-sequence descriptors.

A step is a list of entries (a live request's cache, its next tokens, the places among them
whose logits are wanted). Prompt portions of any length and single decoded tokens sit side by
side; the tokens of all entries are laid end to end:

  token_ids [T], positions [T]        the tokens and their absolute positions
  cu_q [S + 1]                        entry s owns rows cu_q[s] .. cu_q[s + 1]
  ctx_len [S]                         the request's length once this step's tokens are in
  state_slots [S]                     the request's slot of fixed-size state
  logit_rows [R]                      flat rows whose logits are returned, in entry / want order
  row_slots [R]                       the state slot of the request that each of those rows belongs to
  token_src [T]                       state slot whose record holds the token (still on the device), or -1
  per paged cache group:
    block_table [S, W]                page ids, padded with the group's scratch page
    slot_map [T]                      page * page_tokens + slot where the token's K and V go
  per query-tile size asked for by a mixer:
    tile_seq, tile_q0 [tiles]         the list of (entry, first query of the tile)

Everything is int32 and packed into one pinned host buffer, so a step costs one host-to-device
copy whatever the number of layers (as layover/model.py:6-8 and layover/kv/paged_cache.py:143-152
do for their two kinds of step). With a `capacity`, the device buffer has a fixed size and
address (what a captured CUDA graph needs) and unused rows are padded with entries of one token
that read and write only the scratch page and the scratch slot.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheManager, SequenceCache


DEVICE_TOKEN = -1   # a token id that means: the request's last sampled token, as its record on the device has it


@dataclass
class StepEntry:
    """`tokens` are token ids. `[DEVICE_TOKEN]` stands for the token that was last sampled for this
    request: it is in the request's record on the device (where the sampling kernel put it), so a
    step can be launched before the host has read it."""
    seq: SequenceCache
    tokens: list[int]
    want: list[int] = field(default_factory=list)


@dataclass
class GroupBatch:
    block_table: torch.Tensor
    slot_map: torch.Tensor


@dataclass
class QueryTiles:
    tile_seq: torch.Tensor
    tile_q0: torch.Tensor
    count: int


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    cu_q: torch.Tensor
    ctx_len: torch.Tensor
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    n_logit_rows: int
    row_slots: torch.Tensor      # per logit row: the state slot of its request
    token_src: torch.Tensor      # per token: the state slot whose record holds it, or -1
    device_tokens: bool          # whether any token comes from the device
    groups: list[GroupBatch]
    tiles: dict[int, QueryTiles]
    # a mixed step (prompt portions beside single tokens) also lists the two kinds apart, so that the
    # single tokens can go through the decode kernels: the sequences with one token, and the query
    # tiles of the others
    decode_seqs: torch.Tensor | None
    n_decode_seqs: int
    decode_max_ctx: int
    portion_tiles: dict[int, QueryTiles]
    # host-side facts for planning launches
    q_lens: list[int]
    ctx_lens: list[int]
    max_q_len: int
    max_ctx: int
    all_decode: bool
    real_seqs: int = 0          # entries that are not padding
    # the longest and the mean context of the sequences with a single token, as the decode attention
    # is to plan for them (a captured step: of the class of steps it is captured for)
    plan_max_ctx: int = 0
    plan_mean_ctx: int = 0
    shared: dict = field(default_factory=dict)   # what parts make once per step and share (rotary tables)


@dataclass(frozen=True)
class BatchCapacity:
    """Fixed sizes of a batch whose buffers must not move (a captured step). `portion == 0`: `seqs`
    entries of one token each, every row's logits wanted, unused rows padded. `portion == N`: one
    entry of exactly N tokens (a prompt portion), with the logits of its last token or none."""
    seqs: int
    table_width: int
    portion: int = 0
    want_last: bool = True

    def __post_init__(self):
        if self.portion and self.seqs != 1:
            raise ValueError("a fixed-capacity prompt portion is a batch of one request")


class _Layout:
    def __init__(self):
        self.size = 0
        self.fields: dict[str, tuple[int, tuple[int, ...]]] = {}

    def add(self, name: str, *shape: int) -> None:
        count = 1
        for s in shape:
            count *= s
        self.fields[name] = (self.size, shape)
        self.size += -(-max(count, 1) // 4) * 4  # keep every array 16-byte aligned


class BatchBuilder:
    """Packs entries into device arrays with one copy. Keeps a small ring of pinned buffers."""

    def __init__(self, cache: CacheManager, device: torch.device, tile_sizes: tuple[int, ...] = ()):
        self.cache = cache
        self.device = torch.device(device)
        self.tile_sizes = tuple(sorted(set(tile_sizes)))
        self._ring: list[tuple[torch.Tensor, torch.cuda.Event | None]] = []
        self._next = 0

    def _pinned(self, size: int) -> tuple[torch.Tensor, int]:
        if self.device.type != "cuda":
            return torch.empty(size, dtype=torch.int32), -1
        if len(self._ring) < 4:
            self._ring.append((torch.empty(max(size, 4096), dtype=torch.int32, pin_memory=True), None))
        index = self._next % len(self._ring)
        self._next += 1
        buffer, event = self._ring[index]
        if event is not None:
            event.synchronize()
        if buffer.numel() < size:
            buffer = torch.empty(size * 2, dtype=torch.int32, pin_memory=True)
        self._ring[index] = (buffer, None)
        return buffer[:size], index

    def build(self, entries: list[StepEntry], capacity: BatchCapacity | None = None,
              device_buffer: torch.Tensor | None = None, plan_ctx: tuple[int, int] | None = None) -> StepBatch:
        cache, page = self.cache, self.cache.block_tokens
        if not entries and capacity is None:
            raise ValueError("a step needs at least one entry")
        real = len(entries)
        n_seqs = capacity.seqs if capacity else real
        if real > n_seqs:
            raise ValueError(f"{real} entries do not fit a batch of {n_seqs}")
        portion = capacity.portion if capacity else 0
        q_lens = [len(e.tokens) for e in entries] + [portion or 1] * (n_seqs - real)
        if min(q_lens) < 1:
            raise ValueError("an entry without tokens")
        starts = [e.seq.num_tokens for e in entries] + [0] * (n_seqs - real)
        ctx_lens = [s + n for s, n in zip(starts, q_lens)]
        n_tokens = sum(q_lens)
        if capacity and n_tokens != n_seqs * (portion or 1):
            raise ValueError(f"a fixed-capacity batch holds {portion or 1} token(s) per entry")
        width = capacity.table_width if capacity else max(1, cache.blocks_for(max(ctx_lens)))
        if not capacity:
            n_rows = sum(len(e.want) for e in entries)
        elif portion:
            n_rows = 1 if capacity.want_last else 0
            if entries and entries[0].want != ([portion - 1] if capacity.want_last else []):
                raise ValueError("this fixed-capacity portion was made for other wanted places")
        else:
            n_rows = n_seqs

        layout = _Layout()
        layout.add("token_ids", n_tokens); layout.add("positions", n_tokens)
        layout.add("cu_q", n_seqs + 1); layout.add("ctx_len", n_seqs); layout.add("state_slots", n_seqs)
        layout.add("logit_rows", n_rows); layout.add("row_slots", n_rows); layout.add("token_src", n_tokens)
        for g in range(len(cache.paged)):
            layout.add(f"table{g}", n_seqs, width); layout.add(f"slots{g}", n_tokens)
        tile_lists = {}
        for size in self.tile_sizes:
            tiles = [(s, q0) for s, n in enumerate(q_lens) for q0 in range(0, n, size)]
            tile_lists[size] = tiles
            layout.add(f"tile_seq{size}", len(tiles)); layout.add(f"tile_q0{size}", len(tiles))
        singles = [s for s, n in enumerate(q_lens) if n == 1]
        mixed = 0 < len(singles) < n_seqs
        portion_lists = {}
        if mixed:
            layout.add("decode_seqs", len(singles))
            for size in self.tile_sizes:
                tiles = [(s, q0) for s, n in enumerate(q_lens) if n > 1 for q0 in range(0, n, size)]
                portion_lists[size] = tiles
                layout.add(f"ptile_seq{size}", len(tiles)); layout.add(f"ptile_q0{size}", len(tiles))

        host, ring_index = self._pinned(layout.size)
        view = host.numpy()

        def put(name, values):
            offset, _ = layout.fields[name]
            view[offset:offset + len(values)] = values

        # per-token arrays are written as whole slices (a prompt portion has thousands of tokens)
        ids_at, pos_at, src_at = (layout.fields[name][0] for name in ("token_ids", "positions", "token_src"))
        rows, row_slots, cu = [], [], [0]
        device_tokens = False
        for index, entry in enumerate(entries):
            n, at = len(entry.tokens), cu[-1]
            for w in entry.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {entry.seq.request_id!r}: wanted place {w} is outside its {n} tokens")
                rows.append(at + w)
                row_slots.append(entry.seq.slot)
            view[ids_at + at: ids_at + at + n] = entry.tokens
            view[pos_at + at: pos_at + at + n] = np.arange(starts[index], starts[index] + n, dtype=np.int32)
            view[src_at + at: src_at + at + n] = -1
            if n == 1 and entry.tokens[0] < 0:          # the request's newest token is in its record on the device
                view[ids_at + at] = 0
                view[src_at + at] = entry.seq.slot
                device_tokens = True
            cu.append(at + n)
        for _ in range(n_seqs - real):   # padding rows: token 0 from position 0 on, on the scratch page
            at, n = cu[-1], portion or 1
            view[ids_at + at: ids_at + at + n] = 0
            view[pos_at + at: pos_at + at + n] = np.arange(n, dtype=np.int32)
            view[src_at + at: src_at + at + n] = -1
            cu.append(at + n)
        slots_of_seqs = [e.seq.slot for e in entries] + [cache.scratch_slot] * (n_seqs - real)
        if capacity and not portion:
            rows, row_slots = list(range(n_seqs)), slots_of_seqs
        elif capacity and not entries:
            rows, row_slots = [portion - 1] * n_rows, [cache.scratch_slot] * n_rows
        put("cu_q", cu); put("ctx_len", ctx_lens)
        put("state_slots", slots_of_seqs)
        put("logit_rows", rows); put("row_slots", row_slots)
        for g, group in enumerate(cache.paged):
            scratch = group.scratch_page
            offset, _ = layout.fields[f"table{g}"]
            slots_at = layout.fields[f"slots{g}"][0]
            for index in range(n_seqs):
                row = view[offset + index * width: offset + (index + 1) * width]
                row[:] = scratch
                if index < real:
                    entry = entries[index]
                    blocks = entry.seq.tables[g].blocks
                    needed = cache.blocks_for(ctx_lens[index])
                    if needed > len(blocks) or needed > width:
                        raise ValueError(
                            f"request {entry.seq.request_id!r}: {ctx_lens[index]} tokens need {needed} pages, "
                            f"its table has {len(blocks)} and the batch is {width} wide")
                    row[:needed] = blocks[:needed]
                    cache.check_row(g, row[:needed], entry.seq.request_id)     # no bad page id reaches a kernel
                    where = np.arange(starts[index], ctx_lens[index], dtype=np.int64)
                    view[slots_at + cu[index]: slots_at + cu[index + 1]] = row[where // page] * page + where % page
                else:
                    where = np.arange(q_lens[index], dtype=np.int64)
                    view[slots_at + cu[index]: slots_at + cu[index + 1]] = scratch * page + where % page
        for size, tiles in tile_lists.items():
            put(f"tile_seq{size}", [t[0] for t in tiles]); put(f"tile_q0{size}", [t[1] for t in tiles])
        if mixed:
            put("decode_seqs", singles)
            for size, tiles in portion_lists.items():
                put(f"ptile_seq{size}", [t[0] for t in tiles]); put(f"ptile_q0{size}", [t[1] for t in tiles])

        if device_buffer is not None:
            if device_buffer.numel() < layout.size:
                raise ValueError("the fixed device buffer is too small for this batch")
            device = device_buffer[:layout.size]
            device.copy_(host, non_blocking=True)
        else:
            device = host.to(self.device, non_blocking=True)
        if ring_index >= 0:
            event = torch.cuda.Event()
            event.record()
            self._ring[ring_index] = (self._ring[ring_index][0], event)

        def get(name):
            offset, shape = layout.fields[name]
            count = 1
            for s in shape:
                count *= s
            return device[offset:offset + count].view(*shape)

        return StepBatch(
            n_tokens=n_tokens, n_seqs=n_seqs,
            token_ids=get("token_ids"), positions=get("positions"), cu_q=get("cu_q"), ctx_len=get("ctx_len"),
            state_slots=get("state_slots"), logit_rows=get("logit_rows"), n_logit_rows=n_rows,
            row_slots=get("row_slots"), token_src=get("token_src"), device_tokens=device_tokens,
            groups=[GroupBatch(get(f"table{g}"), get(f"slots{g}")) for g in range(len(cache.paged))],
            tiles={size: QueryTiles(get(f"tile_seq{size}"), get(f"tile_q0{size}"), len(tiles))
                   for size, tiles in tile_lists.items()},
            decode_seqs=get("decode_seqs") if mixed else None, n_decode_seqs=len(singles) if mixed else 0,
            decode_max_ctx=max((ctx_lens[s] for s in singles), default=0) if mixed else 0,
            portion_tiles={size: QueryTiles(get(f"ptile_seq{size}"), get(f"ptile_q0{size}"), len(tiles))
                           for size, tiles in portion_lists.items()},
            q_lens=q_lens, ctx_lens=ctx_lens, max_q_len=max(q_lens), max_ctx=max(ctx_lens),
            all_decode=max(q_lens) == 1, real_seqs=real,
            plan_max_ctx=plan_ctx[0] if plan_ctx else max((ctx_lens[s] for s in singles), default=0),
            plan_mean_ctx=plan_ctx[1] if plan_ctx else (sum(ctx_lens[s] for s in singles) // len(singles) if singles else 0),
        )

    @staticmethod
    def buffer_size(capacity: BatchCapacity, n_groups: int, tile_sizes: tuple[int, ...]) -> int:
        """Upper bound of the int32 words a fixed-capacity batch takes."""
        pad = lambda n: -(-max(n, 1) // 4) * 4
        s = capacity.seqs
        t = s * (capacity.portion or 1)
        total = 3 * pad(t) + pad(s + 1) + 4 * pad(s)
        total += n_groups * (pad(s * capacity.table_width) + pad(t))
        total += sum(2 * pad(s * -(-(capacity.portion or 1) // size)) for size in set(tile_sizes))
        return total
