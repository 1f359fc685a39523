"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; state slots; the batch builder's descriptors."""

import random

import pytest
import torch

from layover_b200.cache import BlockAllocator, CacheManager, OutOfBlocks
from layover_b200.engine.batch import BatchBuilder, BatchCapacity, StepEntry
from layover_b200.parts.base import PagedKVNeed, StateNeed

FULL = PagedKVNeed(2, 16, None)
WINDOW = PagedKVNeed(2, 16, 10)
STATE = StateNeed((3, 4), torch.float32)


def manager(needs, blocks=12, page=4, device=None, max_requests=6):
    return CacheManager([(i, n, None) for i, n in enumerate(needs)], blocks, page, torch.float32, device, max_requests)


def test_allocator_hands_out_all_or_nothing_and_refuses_double_free():
    a = BlockAllocator(4)
    got = a.alloc(3)
    assert got == [0, 1, 2] and a.num_free == 1
    with pytest.raises(OutOfBlocks):
        a.alloc(2)
    assert a.num_free == 1                      # nothing changed
    a.free(1)
    assert a.alloc(1) == [1]                    # the page freed last is used again first
    a.free(0)
    with pytest.raises(ValueError, match="not allocated"):
        a.free(0)
    with pytest.raises(ValueError, match="outside"):
        a.free(9)
    a.check()


def test_layers_with_the_same_need_share_a_group_and_others_do_not():
    m = manager([FULL, WINDOW, FULL, STATE, WINDOW])
    assert len(m.paged) == 2 and len(m.states) == 1
    assert m.paged[0].entries == [0, 2] and m.paged[1].entries == [1, 4] and m.states[0].entries == [3]
    assert (m.view(2).group, m.view(2).layer) == (0, 1)
    assert m.view(3).kind == "state"


def test_an_entry_may_read_another_entrys_pages():
    m = CacheManager([(0, FULL, None), (1, FULL, None), (2, FULL, 0)], 4, 4, torch.float32, "cpu", 2)
    assert m.paged[0].pool.shape[0] == 2              # the reader owns no pages
    reader, owner = m.view(2), m.view(0)
    assert reader.writes is False and reader.layer == owner.layer
    assert reader.k_pool.data_ptr() == owner.k_pool.data_ptr()
    with pytest.raises(ValueError, match="reads the cache"):
        CacheManager([(0, None, None), (1, FULL, 0)], 4, 4, torch.float32, None, 2)


def test_grow_commit_close_and_reuse():
    m = manager([FULL], blocks=5, page=4)
    a = m.open("a")
    m.grow(a, 9); m.commit(a, 9)
    assert a.tables[0].blocks == [0, 1, 2] and a.num_tokens == 9
    b = m.open("b")
    with pytest.raises(OutOfBlocks):
        m.grow(b, 12)                                # three pages wanted, two free: nothing taken
    assert m.paged[0].allocator.num_free == 2 and b.tables[0].blocks == []
    m.grow(b, 8); m.commit(b, 8)
    m.close(a)
    c = m.open("c")
    m.grow(c, 4)
    assert c.tables[0].blocks == [2]                 # a's last page, used again
    m.check()
    with pytest.raises(ValueError, match="closed before"):
        m.close(a)
    with pytest.raises(ValueError, match="already open"):
        m.open("b")
    m.close(b); m.close(c)
    assert m.num_free == 5
    m.check()


def test_a_window_gives_pages_back_and_takes_them_again():
    m = manager([WINDOW], blocks=6, page=4)     # window 10: a query at p sees keys > p - 10
    s = m.open("s")
    held_most = 0
    for total in range(1, 60):
        m.grow(s, total); m.commit(s, total)
        table = s.tables[0]
        first_needed = max(0, total - 10 + 1) // 4
        assert table.first_live == first_needed
        assert all(b == m.paged[0].scratch_page for b in table.blocks[:first_needed])
        assert all(b != m.paged[0].scratch_page for b in table.blocks[first_needed:])
        held_most = max(held_most, m.paged[0].allocator.num_used)
        m.check()
    assert held_most <= 4                            # 60 tokens would need 15 pages without the window
    assert held_most <= m.peak_blocks(0, 60, 1)
    m.close(s)
    assert m.num_free == 6


def test_a_long_portion_through_a_window_skips_pages_nobody_will_read():
    m = manager([WINDOW], blocks=8, page=4)
    s = m.open("s")
    m.grow(s, 3); m.commit(s, 3)
    m.grow(s, 30)                                    # 27 tokens at once: every page is still needed in this step
    assert m.paged[0].allocator.num_used == 8
    m.commit(s, 30)                                  # afterwards only keys >= 21 matter
    assert s.tables[0].first_live == 5 and m.paged[0].allocator.num_used == 3
    m.check_tables(s)
    m.close(s)
    assert m.num_free == 8


def test_state_slots_are_zeroed_and_reused():
    m = manager([STATE, FULL], blocks=4, page=4, device="cpu", max_requests=2)
    a = m.open("a"); b = m.open("b")
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(OutOfBlocks, match="request slots"):
        m.open("c")
    m.view(0).state[a.slot] += 5.0
    m.close(a)
    c = m.open("c")
    assert c.slot == a.slot and float(m.view(0).state[c.slot].abs().sum()) == 0.0
    assert m.states[0].pool.shape == (1, 3, 3, 4)     # entries, slots + scratch, shape


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests_lose_no_page(seed):
    rng = random.Random(seed)
    m = manager([FULL, WINDOW, FULL], blocks=rng.choice([6, 9, 16]), page=rng.choice([2, 4]), max_requests=5)
    live, closed = {}, 0
    for op in range(600):
        choice = rng.random()
        if choice < 0.25 and len(live) < 5:
            name = f"r{op}"
            live[name] = m.open(name)
        elif choice < 0.85 and live:
            name = rng.choice(sorted(live))
            seq = live[name]
            new_total = seq.num_tokens + rng.choice([1, 1, 1, 2, 5, 11])
            before = [g.allocator.num_free for g in m.paged]
            try:
                m.grow(seq, new_total)
            except OutOfBlocks:
                assert [g.allocator.num_free for g in m.paged] == before   # all or nothing, over all groups
            else:
                m.commit(seq, new_total)
        elif live:
            name = rng.choice(sorted(live))
            m.close(live.pop(name)); closed += 1
        m.check()
        for seq in live.values():
            m.check_tables(seq)
    for seq in live.values():
        m.close(seq)
    m.check()
    assert all(g.allocator.num_free == g.allocator.num_blocks for g in m.paged) and closed > 0


def test_batch_descriptors():
    m = manager([FULL, WINDOW], blocks=10, page=4, device="cpu")
    a, b = m.open("a"), m.open("b")
    m.grow(a, 6); m.commit(a, 6)
    entries = [StepEntry(a, [7, 8, 9], [0, 2]), StepEntry(b, [1] * 5, [4])]
    for e in entries:
        m.grow(e.seq, e.seq.num_tokens + len(e.tokens))
    batch = BatchBuilder(m, "cpu", (2, 4)).build(entries)
    assert batch.token_ids.tolist() == [7, 8, 9, 1, 1, 1, 1, 1]
    assert batch.positions.tolist() == [6, 7, 8, 0, 1, 2, 3, 4]
    assert batch.cu_q.tolist() == [0, 3, 8] and batch.ctx_len.tolist() == [9, 5]
    assert batch.logit_rows.tolist() == [0, 2, 7] and batch.n_logit_rows == 3
    assert batch.state_slots.tolist() == [a.slot, b.slot]
    table = batch.groups[0].block_table
    assert table.shape == (2, 3) and table[0].tolist() == a.tables[0].blocks[:3]
    assert table[1].tolist() == b.tables[0].blocks[:2] + [m.paged[0].scratch_page]
    pages = a.tables[0].blocks
    assert batch.groups[0].slot_map.tolist()[:3] == [pages[1] * 4 + 2, pages[1] * 4 + 3, pages[2] * 4 + 0]
    tiles = batch.tiles[2]
    assert list(zip(tiles.tile_seq.tolist(), tiles.tile_q0.tolist())) == [(0, 0), (0, 2), (1, 0), (1, 2), (1, 4)]
    assert batch.tiles[4].count == 3 and not batch.all_decode and batch.max_ctx == 9
    with pytest.raises(ValueError, match="wanted place"):
        BatchBuilder(m, "cpu").build([StepEntry(a, [1], [1])])


def test_a_mixed_step_lists_single_tokens_and_portions_apart():
    m = manager([FULL], blocks=20, page=4, device="cpu")
    a, b, c, d = (m.open(name) for name in "abcd")
    for seq, held in ((a, 6), (c, 9)):
        m.grow(seq, held); m.commit(seq, held)
    entries = [StepEntry(a, [7], [0]), StepEntry(b, [1] * 5, [4]), StepEntry(c, [2], [0]), StepEntry(d, [3, 4], [])]
    for e in entries:
        m.grow(e.seq, e.seq.num_tokens + len(e.tokens))
    batch = BatchBuilder(m, "cpu", (2, 4)).build(entries)
    assert not batch.all_decode and batch.n_decode_seqs == 2 and batch.decode_seqs.tolist() == [0, 2]
    assert batch.decode_max_ctx == 10
    tiles = batch.portion_tiles[2]
    assert list(zip(tiles.tile_seq.tolist(), tiles.tile_q0.tolist())) == [(1, 0), (1, 2), (1, 4), (3, 0)]
    assert batch.portion_tiles[4].count == 3 and batch.tiles[2].count == 6
    # steps of one kind have nothing to tell apart
    only_portions = BatchBuilder(m, "cpu", (2,)).build([StepEntry(b, [5, 5], [])])
    assert only_portions.n_decode_seqs == 0 and only_portions.decode_seqs is None and not only_portions.portion_tiles
    only_singles = BatchBuilder(m, "cpu", (2,)).build([StepEntry(a, [5], [0]), StepEntry(c, [5], [0])])
    assert only_singles.all_decode and only_singles.n_decode_seqs == 0


def test_fixed_capacity_batches_pad_onto_the_scratch_page():
    m = manager([FULL], blocks=10, page=4, device="cpu")
    a = m.open("a")
    m.grow(a, 5); m.commit(a, 5); m.grow(a, 6)
    capacity = BatchCapacity(4, 6)
    buffer = torch.zeros(BatchBuilder.buffer_size(capacity, 1, (16,)), dtype=torch.int32)
    batch = BatchBuilder(m, "cpu", (16,)).build([StepEntry(a, [3], [0])], capacity, buffer)
    scratch = m.paged[0].scratch_page
    assert batch.n_seqs == 4 and batch.real_seqs == 1 and batch.all_decode
    assert batch.ctx_len.tolist() == [6, 1, 1, 1] and batch.positions.tolist() == [5, 0, 0, 0]
    assert batch.groups[0].block_table.shape == (4, 6)
    assert batch.groups[0].block_table[1].tolist() == [scratch] * 6
    assert batch.groups[0].slot_map.tolist()[1:] == [scratch * 4] * 3
    assert batch.state_slots.tolist()[1:] == [m.scratch_slot] * 3
    assert batch.token_ids.data_ptr() == buffer.data_ptr()      # the descriptors sit at the fixed address
    with pytest.raises(ValueError, match=r"1 token\(s\) per entry"):
        BatchBuilder(m, "cpu").build([StepEntry(a, [3, 4], [0])], capacity, buffer)


def test_a_fixed_capacity_prompt_portion():
    """One request with exactly the capacity's tokens, at the fixed address, with the last token's
    logits or none; with no request at all (what a capture runs) the tokens lie on the scratch page."""
    m = manager([FULL], blocks=12, page=4, device="cpu")
    a = m.open("a")
    m.grow(a, 3); m.commit(a, 3); m.grow(a, 13)
    capacity = BatchCapacity(1, 8, portion=10, want_last=True)
    words = BatchBuilder.buffer_size(capacity, 1, (4, 16))
    buffer = torch.zeros(words, dtype=torch.int32)
    builder = BatchBuilder(m, "cpu", (4, 16))
    tokens = list(range(20, 30))
    batch = builder.build([StepEntry(a, tokens, [9])], capacity, buffer)
    assert batch.n_tokens == 10 and batch.n_seqs == 1 and not batch.all_decode and batch.n_logit_rows == 1
    assert batch.token_ids.tolist() == tokens and batch.positions.tolist() == list(range(3, 13))
    assert batch.ctx_len.tolist() == [13] and batch.logit_rows.tolist() == [9] and batch.row_slots.tolist() == [a.slot]
    assert batch.groups[0].block_table.shape == (1, 8)
    blocks = a.tables[0].blocks
    assert batch.groups[0].slot_map.tolist() == [blocks[p // 4] * 4 + p % 4 for p in range(3, 13)]
    assert batch.tiles[4].count == 3 and batch.tiles[4].tile_q0.tolist() == [0, 4, 8] and batch.tiles[16].count == 1
    assert batch.token_ids.data_ptr() == buffer.data_ptr()
    layout_words = batch.tiles[16].tile_q0.data_ptr() - buffer.data_ptr()
    assert layout_words // 4 + 4 <= words
    # the same layout with nothing in it: every table entry and slot is the scratch page's
    scratch = m.paged[0].scratch_page
    empty = builder.build([], capacity, buffer)
    assert empty.ctx_len.tolist() == [10] and empty.positions.tolist() == list(range(10))
    assert set(empty.groups[0].block_table.flatten().tolist()) == {scratch}
    assert all(slot // 4 == scratch for slot in empty.groups[0].slot_map.tolist())
    assert empty.row_slots.tolist() == [m.scratch_slot] and empty.logit_rows.tolist() == [9]
    assert empty.positions.data_ptr() == batch.positions.data_ptr()
    # other sizes and other wanted places are refused
    with pytest.raises(ValueError, match=r"10 token\(s\) per entry"):
        builder.build([StepEntry(a, tokens[:9], [8])], capacity, buffer)
    with pytest.raises(ValueError, match="other wanted places"):
        builder.build([StepEntry(a, tokens, [])], capacity, buffer)
    none_wanted = builder.build([StepEntry(a, tokens, [])], BatchCapacity(1, 8, portion=10, want_last=False), buffer)
    assert none_wanted.n_logit_rows == 0
    with pytest.raises(ValueError, match="batch of one request"):
        BatchCapacity(2, 8, portion=10)


def test_a_batch_carries_the_contexts_its_decode_attention_plans_for():
    """The longest and the mean context of the entries with a single token (the others are prompt
    portions); a fixed-capacity batch takes them from the class of steps it stands for."""
    m = manager([FULL], blocks=40, page=4, device="cpu")
    seqs = []
    for name, held in (("a", 30), ("b", 6), ("c", 11)):
        seq = m.open(name)
        m.grow(seq, held); m.commit(seq, held); m.grow(seq, held + 5)
        seqs.append(seq)
    builder = BatchBuilder(m, "cpu", (16,))
    batch = builder.build([StepEntry(seqs[0], [1], [0]), StepEntry(seqs[1], [2], [0]), StepEntry(seqs[2], [3], [0])])
    assert batch.all_decode and (batch.plan_max_ctx, batch.plan_mean_ctx) == (31, (31 + 7 + 12) // 3)
    mixed = builder.build([StepEntry(seqs[0], [1, 2, 3, 4, 5], []), StepEntry(seqs[1], [2], [0]), StepEntry(seqs[2], [3], [0])])
    assert not mixed.all_decode and mixed.n_decode_seqs == 2
    assert (mixed.plan_max_ctx, mixed.plan_mean_ctx) == (12, (7 + 12) // 2)
    capacity = BatchCapacity(4, 16)
    buffer = torch.zeros(BatchBuilder.buffer_size(capacity, 1, (16,)), dtype=torch.int32)
    fixed = builder.build([StepEntry(seqs[1], [2], [0])], capacity, buffer, (64, 32))
    assert (fixed.plan_max_ctx, fixed.plan_mean_ctx) == (64, 32)
