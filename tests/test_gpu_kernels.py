"""Each kernel alone against a plain 32-bit (or 64-bit) reference of the same operation, at sizes
other than the engine's own tiny models: widths that are no power of two, head sizes in steps of
16, any number of heads and groups, pages of several sizes."""

import math
import os

import numpy as np
import pytest
import torch

from conftest import tolerance
from plain_qwen3 import plain_attention, plain_rmsnorm, plain_rope_tables, plain_apply_rope, plain_sample

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from layover_b200 import ops as module
    return module


def close(got, expected, dtype, scale=1.0):
    bound = tolerance(expected.float(), dtype) * scale
    assert (got.float().cpu() - expected.float().cpu()).abs().max().item() <= bound


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab, hidden, tokens", [(50, 96, 7), (1000, 2560, 33), (3, 10, 1)])
def test_embed(dtype, vocab, hidden, tokens):
    table = torch.randn(vocab, hidden, device="cuda").to(dtype)
    ids = torch.randint(0, vocab, (tokens,), device="cuda", dtype=torch.int32)
    out = torch.empty(tokens, hidden, device="cuda", dtype=dtype)
    ops().embed(ids, table, out)
    assert torch.equal(out, table[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, hidden, eps", [(5, 96, 1e-5), (3, 2560, 1e-6), (2, 5000, 1e-6), (17, 16, 1e-3),
                                               (300, 2560, 1e-6), (257, 104, 1e-5), (301, 1024, 1e-6)])
def test_add_rmsnorm(dtype, rows, hidden, eps):
    x = torch.randn(rows, hidden, device="cuda").to(dtype)
    delta = (0.5 * torch.randn(rows, hidden, device="cuda")).to(dtype)
    weight = 1 + 0.2 * torch.randn(hidden, device="cuda")
    summed = (x.float() + delta.float()).to(dtype)
    expected = plain_rmsnorm(summed.cpu(), weight.cpu().to(dtype), eps)
    x_run = x.clone()
    out = torch.empty_like(x)
    ops().add_rmsnorm(x_run, delta, weight.to(dtype).float(), eps, out)
    assert torch.equal(x_run, summed)                                   # the residual stream holds the rounded sum
    close(out, expected, dtype)
    # without a delta, and for picked rows only (x untouched)
    out2 = torch.empty_like(x)
    ops().add_rmsnorm(x.clone(), None, weight.to(dtype).float(), eps, out2)
    close(out2, plain_rmsnorm(x.cpu(), weight.cpu().to(dtype), eps), dtype)
    picked = torch.tensor([rows - 1, 0], device="cuda", dtype=torch.int32)
    x_keep = x.clone()
    out3 = torch.empty(2, hidden, device="cuda", dtype=dtype)
    ops().add_rmsnorm(x_keep, delta, weight.to(dtype).float(), eps, out3, picked)
    assert torch.equal(x_keep, x)
    close(out3, expected[[rows - 1, 0]], dtype)
    if rows >= 256:
        # many rows take the kernel that holds two rows per block in registers: the same bits as
        # the one-row kernel gives for the same rows a few at a time
        x_few, out_few = x.clone(), torch.empty_like(x)
        for start in range(0, rows, 100):
            ops().add_rmsnorm(x_few[start:start + 100], delta[start:start + 100], weight.to(dtype).float(), eps,
                              out_few[start:start + 100])
        assert torch.equal(x_few, x_run) and torch.equal(out_few, out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m, n, k", [(1, 96, 64), (5, 200, 96), (64, 1000, 200), (130, 70, 2560), (3, 5, 7), (33, 257, 130)])
def test_gemm_simt(dtype, m, n, k):
    a = torch.randn(m, k, device="cuda").to(dtype)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(dtype)
    expected = (a.double() @ w.double().T).float()
    out = torch.empty(m, n, device="cuda", dtype=dtype)
    ops().gemm_simt(a, w, out)
    close(out, expected, dtype)
    if dtype == torch.bfloat16:
        wide = torch.empty(m, n, device="cuda", dtype=torch.float32)
        ops().gemm_simt(a, w, wide)
        close(wide, expected, torch.float32, scale=4)
    # strided rows: a view into a wider matrix
    big = torch.randn(m, k + 8, device="cuda").to(dtype)
    out2 = torch.empty(m, n, device="cuda", dtype=dtype)
    ops().gemm_simt(big[:, 4:4 + k], w, out2)
    close(out2, (big[:, 4:4 + k].double() @ w.double().T).float(), dtype)


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    a = torch.randn(70, 200, device="cuda")
    w = torch.randn(96, 200, device="cuda")
    full = torch.empty(70, 96, device="cuda")
    ops().gemm_simt(a, w, full)
    for lo, hi in ((0, 1), (63, 65), (5, 70)):
        part = torch.empty(hi - lo, 96, device="cuda")
        ops().gemm_simt(a[lo:hi].contiguous(), w, part)
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, inter", [(3, 200), (17, 9728), (1, 5)])
def test_swiglu(dtype, tokens, inter):
    gu = (2 * torch.randn(tokens, 2 * inter, device="cuda")).to(dtype)
    out = torch.empty(tokens, inter, device="cuda", dtype=dtype)
    ops().swiglu(gu, out)
    expected = torch.nn.functional.silu(gu[:, :inter].cpu()) * gu[:, inter:].cpu()
    close(out, expected, dtype)
    if inter % 8 == 0:       # gates and ups alternating in blocks of 8 features
        mixed = torch.stack((gu[:, :inter].view(tokens, -1, 8), gu[:, inter:].view(tokens, -1, 8)), dim=2).reshape(tokens, -1)
        out2 = torch.empty_like(out)
        ops().swiglu(mixed.contiguous(), out2, block=8)
        assert torch.equal(out2, out)


def paged_setup(dtype, lengths, kv_heads, dim, page, seed=0, poison=True):
    """Random K and V for sequences of the given lengths, scattered over shuffled pages of a pool
    whose unused slots hold NaN."""
    gen = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page) for n in lengths]
    total = sum(pages_per) + 3
    order = torch.randperm(total - 1, generator=gen).tolist()      # the last page stays unused (scratch)
    fill = float("nan") if poison else 0.0
    k_pool = torch.full((total, kv_heads, page, dim), fill, dtype=dtype)
    v_pool = torch.full((total, kv_heads, page, dim), fill, dtype=dtype)
    width = max(pages_per)
    table = torch.full((len(lengths), width), total - 1, dtype=torch.int32)
    ks, vs = [], []
    for s, n in enumerate(lengths):
        k = torch.randn(n, kv_heads, dim, generator=gen).to(dtype)
        v = torch.randn(n, kv_heads, dim, generator=gen).to(dtype)
        mine = [order.pop() for _ in range(pages_per[s])]
        table[s, :len(mine)] = torch.tensor(mine, dtype=torch.int32)
        for pos in range(n):
            k_pool[mine[pos // page], :, pos % page] = k[pos]
            v_pool[mine[pos // page], :, pos % page] = v[pos]
        ks.append(k); vs.append(v)
    return k_pool.cuda(), v_pool.cuda(), table.cuda(), ks, vs


def run_attention(dtype, lengths, q_lens, q_heads, kv_heads, dim, page, window=0, seed=0, qs=None, kernel="simt",
                  splits=1):
    o = ops()
    k_pool, v_pool, table, ks, vs = paged_setup(dtype, lengths, kv_heads, dim, page, seed)
    gen = torch.Generator().manual_seed(seed + 1)
    if qs is None:
        qs = [torch.randn(n, q_heads, dim, generator=gen).to(dtype) for n in q_lens]
    q = torch.cat(qs).reshape(-1, q_heads * dim).cuda()
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device="cuda")
    ctx = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    bq = o.attention_simt_block_queries() if kernel == "simt" else o.attention_mma_block_queries()
    tiles = [(s, q0) for s, n in enumerate(q_lens) for q0 in range(0, n, bq)]
    tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
    tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    scale = 1.0 / math.sqrt(dim)
    if kernel == "simt":
        o.attention_simt(q, k_pool, v_pool, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads, kv_heads, dim,
                         page, scale, window)
    elif kernel == "prefill":
        o.attention_prefill_bf16(q, k_pool, v_pool, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads,
                                 kv_heads, dim, page, scale, window)
    else:
        assert all(n == 1 for n in q_lens)
        o.attention_decode_bf16(q, k_pool, v_pool, out, table, cu, ctx, None, len(lengths), q_heads, kv_heads, dim,
                                page, scale, window, splits)
    expected = []
    for s, n in enumerate(lengths):
        # the last q_lens[s] positions of a whole-sequence attention in which earlier queries are dummies
        full_q = torch.zeros(n, q_heads, dim, dtype=dtype)
        full_q[n - q_lens[s]:] = qs[s]
        expected.append(plain_attention(full_q, ks[s], vs[s], window or None)[n - q_lens[s]:])
    return out.cpu().view(-1, q_heads, dim), torch.cat(expected), ks, vs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads, kv_heads, dim, page", [(4, 2, 16, 4), (6, 1, 32, 16), (3, 3, 48, 8), (8, 2, 128, 16),
                                                          (2, 1, 256, 16), (5, 5, 80, 2)])
def test_attention_simt_mixed_segments(dtype, q_heads, kv_heads, dim, page):
    # a whole prompt, a portion on top of history, single decoded tokens at page edges
    lengths = [37, 100, page, page + 1, 2 * page - 1, 1, 65]
    q_lens = [37, 9, 1, 1, 1, 1, 2]
    got, expected, _, _ = run_attention(dtype, lengths, q_lens, q_heads, kv_heads, dim, page)
    assert not torch.isnan(got).any()                  # NaN in unused slots and pages did not leak
    close(got, expected, dtype)


@pytest.mark.parametrize("window", [1, 5, 16, 33])
def test_attention_simt_window_edges(window):
    lengths, q_lens = [70, 40, 33], [70, 3, 1]
    got, expected, _, _ = run_attention(torch.float32, lengths, q_lens, 4, 2, 32, 8, window=window)
    close(got, expected, torch.float32)


@pytest.mark.parametrize("far_key", [0, 15, 16, 17, 255, 256, 499, 500, 511])
def test_attention_finds_one_far_key_among_hundreds(far_key):
    """Random keys all look alike to a random query; here one key is made to stand out, so that a
    kernel that skips or misplaces it (a page's edge, the first or last key) gives a different answer."""
    dim, n = 64, 512
    dtype = torch.float32
    gen = torch.Generator().manual_seed(3)
    direction = torch.randn(dim, generator=gen)
    direction /= direction.norm()
    q = (direction * 40.0).view(1, 1, dim)
    k_pool, v_pool, table, ks, vs = paged_setup(dtype, [n], 1, dim, 16, seed=4)
    page = int(table[0, far_key // 16])
    k_pool[page, 0, far_key % 16] = (direction * 40.0).cuda()
    marker = torch.full((dim,), 7.0)
    v_pool[page, 0, far_key % 16] = marker.cuda()
    o = ops()
    out = torch.empty(1, dim, device="cuda")
    one = torch.ones(1, dtype=torch.int32, device="cuda")
    o.attention_simt(q.view(1, dim).cuda(), k_pool, v_pool, out, table, torch.tensor([0, 1], dtype=torch.int32, device="cuda"),
                     n * one, 0 * one, 0 * one, 1, 1, 1, dim, 16, 1.0 / math.sqrt(dim))
    assert (out.cpu() - marker).abs().max() < 1e-3     # score 200 against |scores| of a few: all weight on that key


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads, kv_heads, dim, page", [(4, 2, 16, 4), (6, 1, 32, 16), (32, 8, 128, 16), (2, 2, 256, 8),
                                                          (3, 1, 80, 16)])
def test_qk_norm_rope_kv(dtype, q_heads, kv_heads, dim, page):
    o = ops()
    tokens, eps, theta = 11, 1e-5, 50000.0
    gen = torch.Generator().manual_seed(dim)
    qkv = torch.randn(tokens, (q_heads + 2 * kv_heads) * dim, generator=gen).to(dtype)
    qn = (1 + 0.2 * torch.randn(dim, generator=gen)).to(dtype)
    kn = (1 + 0.2 * torch.randn(dim, generator=gen)).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 7, 8, 9, 4000, 39999], dtype=torch.int32)
    pages = 6
    slots = torch.randperm(pages * page, generator=gen)[:tokens].to(torch.int32)
    k_pool = torch.zeros(pages, kv_heads, page, dim, dtype=dtype, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty(tokens, q_heads * dim, dtype=dtype, device="cuda")
    inv_freq = (1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))).cuda()
    table = torch.empty(tokens, 2, dim // 2, device="cuda")
    o.rope_table(positions.cuda(), inv_freq, table)
    o.qk_norm_rope_kv(qkv.cuda(), q_out, k_pool, v_pool, qn.float().cuda(), kn.float().cuda(), table,
                      slots.cuda(), q_heads, kv_heads, dim, page, eps)
    heads = qkv.view(tokens, q_heads + 2 * kv_heads, dim)
    cos, sin = plain_rope_tables(positions, dim, theta, dtype)
    q_ref = plain_apply_rope(plain_rmsnorm(heads[:, :q_heads], qn, eps), cos, sin)
    k_ref = plain_apply_rope(plain_rmsnorm(heads[:, q_heads:q_heads + kv_heads], kn, eps), cos, sin)
    v_ref = heads[:, q_heads + kv_heads:]
    # positions up to 4e4 turn a rounding of the 32-bit angle into ~1e-3 of the cosine: compare loosely there
    close(q_out.view(tokens, q_heads, dim), q_ref, dtype, scale=1.0 if dtype == torch.bfloat16 else 40.0)
    for t in range(tokens):
        pg, sl = int(slots[t]) // page, int(slots[t]) % page
        close(k_pool[pg, :, sl], k_ref[t], dtype, scale=1.0 if dtype == torch.bfloat16 else 40.0)
        assert torch.equal(v_pool[pg, :, sl].cpu(), v_ref[t])
    written = torch.zeros(pages * page, dtype=torch.bool)
    written[slots.long()] = True
    untouched = k_pool.permute(0, 2, 1, 3).reshape(pages * page, -1)[~written.cuda()]
    assert float(untouched.abs().sum()) == 0.0          # nothing outside the given slots was written


def test_qk_norm_rope_small_positions_are_tight():
    o = ops()
    dim, theta = 64, 10000.0
    x = torch.randn(4, 3 * dim)
    positions = torch.tensor([0, 1, 5, 17], dtype=torch.int32)
    inv_freq = (1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))).cuda()
    q_out = torch.empty(4, dim, device="cuda")
    k_pool = torch.zeros(1, 1, 4, dim, device="cuda"); v_pool = torch.zeros_like(k_pool)
    table = torch.empty(4, 2, dim // 2, device="cuda")
    o.rope_table(positions.cuda(), inv_freq, table)
    angles = positions.float()[:, None] * inv_freq.cpu()[None, :]
    assert (table[:, 0].cpu() - angles.cos()).abs().max() < 2e-6 and (table[:, 1].cpu() - angles.sin()).abs().max() < 2e-6
    o.qk_norm_rope_kv(x.cuda(), q_out, k_pool, v_pool, None, None, table,
                      torch.arange(4, dtype=torch.int32, device="cuda"), 1, 1, dim, 4, 0.0)
    cos, sin = plain_rope_tables(positions, dim, theta, torch.float32)
    expected = plain_apply_rope(x.view(4, 3, dim)[:, :1], cos, sin)
    assert (q_out.cpu().view(4, 1, dim) - expected).abs().max() < 2e-6


def test_refused_sizes_raise_instead_of_computing():
    o = ops()
    x = torch.zeros(2, 3 * 258, device="cuda")
    with pytest.raises(ValueError, match="unsupported size"):
        o.qk_norm_rope_kv(x, torch.zeros(2, 258, device="cuda"), None, None, None, None, None, None, 1, 1, 258, 4, 0.0)
    with pytest.raises(ValueError, match="contiguous"):
        o.swiglu(torch.zeros(4, 8, device="cuda").t(), torch.zeros(8, 2, device="cuda"))
    with pytest.raises(Exception, match="CUDA"):
        o.embed(torch.zeros(2, dtype=torch.int32), torch.zeros(3, 4), torch.zeros(2, 4))


def make_records(o, temperatures, seeds, counts, slots_total=None):
    """Per-request records as the cache manager holds them, one row per request (row r = slot r)."""
    from layover_b200.sampling.sampler import SamplingParams, request_record
    rows = [request_record(SamplingParams(float(t), int(s))) for t, s in zip(temperatures, seeds)]
    records = torch.zeros((slots_total or len(rows), o.RECORD_WORDS), dtype=torch.int64)
    records[: len(rows)] = torch.tensor(rows, dtype=torch.int64)
    records[: len(rows), o.RECORD_COUNT] = torch.tensor([c - (1 << 32) if c >= (1 << 31) else c for c in counts])
    return records.to(torch.int32).cuda()


@pytest.mark.parametrize("vocab", [7, 512, 151936, 1000])
def test_sampling_matches_the_plain_rule(vocab):
    o = ops()
    rows = 6
    gen = torch.Generator().manual_seed(vocab)
    logits = torch.randn(rows, vocab, generator=gen) * 3
    logits[0, vocab // 2] = logits[0].max() + 1          # a clear maximum
    logits[1, 3] = logits[1, 5] = logits[1].max() + 2    # equal maxima: the first wins
    temperature = [0.0, 0.0, 0.8, 1.5, 0.8, 0.3]
    seeds = [0, 0, 1234, 0xFFFFFFFF12345678, 1234, 99]
    steps = [0, 0, 0, 7, 1, 4000000000]
    # the rows' requests sit in slots 5, 4, .. 0 of a pool of 9: the kernel must go through row_slots
    records = make_records(o, temperature[::-1], seeds[::-1], steps[::-1], slots_total=9)
    before = records.clone()
    row_slots = torch.tensor([5, 4, 3, 2, 1, 0], dtype=torch.int32, device="cuda")
    positions = torch.arange(40, 52, dtype=torch.int32, device="cuda")
    logit_rows = torch.tensor([1, 3, 5, 7, 9, 11], dtype=torch.int32, device="cuda")
    tokens = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    o.sample(logits.cuda(), tokens, records, row_slots, positions, logit_rows)
    expected = [plain_sample(logits[r].numpy(), temperature[r], seeds[r], steps[r]) for r in range(rows)]
    assert tokens.tolist() == expected
    assert expected[0] == vocab // 2 and expected[1] == 3
    # what the kernel leaves in the records: the token, the counter one further, the position; nothing else
    after = records.cpu().to(torch.int64)
    for r in range(rows):
        slot = 5 - r
        assert after[slot, o.RECORD_LAST_TOKEN] == expected[r]
        assert (after[slot, o.RECORD_COUNT] & 0xFFFFFFFF) == (steps[r] + 1) & 0xFFFFFFFF
        assert after[slot, o.RECORD_POSITION] == 40 + 2 * r + 1 + 2
    untouched = [o.RECORD_SEED_LO, o.RECORD_SEED_HI, o.RECORD_TEMPERATURE, 6, 7]
    assert torch.equal(after[:, untouched], before.cpu().to(torch.int64)[:, untouched])
    assert torch.equal(after[6:], before.cpu().to(torch.int64)[6:])
    greedy = torch.empty(rows, dtype=torch.int32, device="cuda")
    o.sample(logits.cuda(), greedy)
    assert greedy.tolist() == logits.argmax(-1).tolist()


def test_sampling_carries_other_kernels_error_words_behind_the_tokens():
    o = ops()
    words = torch.tensor([0, 5], dtype=torch.int32, device="cuda")        # stand-ins for two libraries' error words
    status = torch.tensor([words.data_ptr(), words.data_ptr() + 4], dtype=torch.int64, device="cuda")
    logits = torch.randn(3, 40, device="cuda")
    tokens = torch.full((5,), -1, dtype=torch.int32, device="cuda")
    o.sample(logits, tokens, status=status)
    assert tokens.tolist() == logits.argmax(-1).tolist() + [0, 5]
    with pytest.raises(ValueError, match="tokens must hold"):
        o.sample(logits, torch.empty(3, dtype=torch.int32, device="cuda"), status=status)


def test_embedding_takes_tokens_from_the_requests_records():
    o = ops()
    table = torch.randn(50, 24, device="cuda").to(torch.bfloat16)
    records = make_records(o, [0.0] * 4, [0] * 4, [0] * 4)
    records[:, o.RECORD_LAST_TOKEN] = torch.tensor([7, 49, 0, 12], dtype=torch.int32, device="cuda")
    ids = torch.tensor([3, 0, 0, 9, 0], dtype=torch.int32, device="cuda")
    source = torch.tensor([-1, 1, 3, -1, 0], dtype=torch.int32, device="cuda")
    out = torch.empty(5, 24, dtype=torch.bfloat16, device="cuda")
    o.embed(ids, table, out, source, records)
    assert torch.equal(out, table[torch.tensor([3, 49, 12, 9, 7], device="cuda")])
    o.embed(ids, table, out)
    assert torch.equal(out, table[ids.long()])
    odd = torch.randn(50, 23, device="cuda")                                  # rows that are no multiple of 16 bytes
    out = torch.empty(5, 23, device="cuda")
    o.embed(ids, odd, out, source, records)
    assert torch.equal(out, odd[torch.tensor([3, 49, 12, 9, 7], device="cuda")])


def test_sampling_follows_the_distribution():
    o = ops()
    probs = torch.tensor([0.5, 0.25, 0.125, 0.125])
    n = 4000
    logits = probs.log().repeat(n, 1).cuda()
    tokens = torch.empty(n, dtype=torch.int32, device="cuda")
    records = make_records(o, [1.0], [77], [0]).repeat(n, 1)
    records[:, o.RECORD_COUNT] = torch.arange(n, dtype=torch.int32, device="cuda")
    o.sample(logits, tokens, records.contiguous(), torch.arange(n, dtype=torch.int32, device="cuda"))
    freq = torch.bincount(tokens.long().cpu(), minlength=4).float() / n
    assert (freq - probs).abs().max() < 0.03


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m, n, k", [
    (1, 96, 64), (8, 2560, 4096), (16, 6144, 2560), (17, 200, 96), (33, 1000, 200), (64, 2560, 9728), (100, 392, 136),
    (128, 256, 64), (129, 96, 64), (300, 200, 96), (2048, 640, 2560), (257, 1000, 264), (5, 8, 8), (8, 151936, 64),
    # 512 tokens and more on wide weights: pairs of blocks on tiles of 256 x 256 (whole tiles, ragged
    # edges on both sides, a last round split along K, several rounds)
    (512, 256, 64), (513, 300, 136), (1000, 2560, 4096), (2048, 6144, 2560), (700, 520, 264), (4096, 10240, 512),
])
def test_gemm_tcgen05(out_dtype, m, n, k):
    o = ops()
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
    expected = (a.double() @ w.double().T).float()
    assert o.gemm_tcgen05_supports(a, w)
    for _ in range(2):                                   # twice: a split-K tile counter must be back at zero
        out = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
        o.gemm_tcgen05(a, w, out)
        assert o.gemm_status() == 0
        assert not torch.isnan(out).any()
        close(out, expected, out_dtype if out_dtype == torch.bfloat16 else torch.float32, scale=1.0 if out_dtype == torch.bfloat16 else 8.0)


def test_gemm_tcgen05_strided_views_and_fallback():
    o = ops()
    big = torch.randn(40, 512, device="cuda").to(torch.bfloat16)
    w = torch.randn(72, 128, device="cuda").to(torch.bfloat16) / 11
    view = big[:, 128:256]                               # rows 1024 bytes apart, start 256 bytes in
    out = torch.empty(40, 72, device="cuda", dtype=torch.bfloat16)
    o.gemm_bf16(view, w, out)
    close(out, (view.double() @ w.double().T).float(), torch.bfloat16)
    wide = torch.empty(40, 80, device="cuda", dtype=torch.bfloat16)
    o.gemm_bf16(view, w, wide[:, 3:75])                  # an output view that no vector store may touch
    close(wide[:, 3:75], (view.double() @ w.double().T).float(), torch.bfloat16)
    odd = torch.randn(9, 100, device="cuda").to(torch.bfloat16)[:, :99]   # K = 99: TMA cannot address it
    w_odd = torch.randn(20, 99, device="cuda").to(torch.bfloat16)
    assert not o.gemm_tcgen05_supports(odd, w_odd)
    out = torch.empty(9, 20, device="cuda", dtype=torch.bfloat16)
    o.gemm_bf16(odd, w_odd, out)
    close(out, (odd.double() @ w_odd.double().T).float(), torch.bfloat16)
    assert o.gemm_status() == 0


@pytest.mark.parametrize("q_heads, kv_heads, dim, page", [(4, 2, 16, 4), (6, 1, 32, 16), (3, 3, 48, 8), (32, 8, 128, 16),
                                                          (2, 1, 256, 16), (5, 5, 80, 2), (16, 2, 64, 32), (8, 2, 144, 16)])
def test_attention_prefill_bf16(q_heads, kv_heads, dim, page):
    lengths = [37, 300, page, page + 1, 2 * page - 1, 1, 65, 64, 200]
    q_lens = [37, 129, 1, 1, 1, 1, 2, 64, 70]
    got, expected, _, _ = run_attention(torch.bfloat16, lengths, q_lens, q_heads, kv_heads, dim, page, kernel="prefill")
    assert not torch.isnan(got).any()
    close(got, expected, torch.bfloat16)


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_prefill_bf16_window(window):
    got, expected, _, _ = run_attention(torch.bfloat16, [270, 140, 33], [270, 3, 1], 4, 2, 32, 8, window=window, kernel="prefill")
    close(got, expected, torch.bfloat16)


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("q_heads, kv_heads, dim, page", [(4, 2, 16, 4), (6, 1, 32, 16), (32, 8, 128, 16), (2, 1, 256, 16),
                                                          (16, 1, 64, 8), (5, 5, 80, 2)])
def test_attention_decode_bf16(q_heads, kv_heads, dim, page, splits):
    lengths = [1, 2, page, page + 1, 63, 64, 65, 127, 128, 129, 700, 1000, 257]
    for _ in range(2):                                 # twice: the split counters must be back at zero
        got, expected, _, _ = run_attention(torch.bfloat16, lengths, [1] * len(lengths), q_heads, kv_heads, dim, page,
                                            kernel="decode", splits=splits)
        assert not torch.isnan(got).any()
        close(got, expected, torch.bfloat16)


@pytest.mark.parametrize("splits", [2, 4, 8])
@pytest.mark.parametrize("q_heads, kv_heads", [(32, 8), (16, 1), (3, 1), (2, 2), (12, 1)])
def test_attention_decode_bf16_splits_as_clusters(q_heads, kv_heads, splits):
    """Head size 128 with 2, 4 or 8 splits: the splits of a (sequence, KV head) run as a thread-block
    cluster and merge through distributed shared memory; groups of 1 to 16 heads, shares of the
    outputs that do not divide evenly, splits without a single tile (short contexts), a window."""
    lengths = [1, 2, 17, 63, 64, 65, 127, 128, 129, 700, 1000, 257, 513]
    for window in (0, 100):
        for _ in range(2):
            got, expected, _, _ = run_attention(torch.bfloat16, lengths, [1] * len(lengths), q_heads, kv_heads, 128, 16,
                                                window=window, kernel="decode", splits=splits)
            assert not torch.isnan(got).any()
            close(got, expected, torch.bfloat16)


@pytest.mark.parametrize("splits", [1, 2, 3, 4])
@pytest.mark.parametrize("q_heads, kv_heads", [(32, 8), (8, 1), (3, 3)])
def test_attention_decode_bf16_with_two_stages(q_heads, kv_heads, splits):
    """The variant with two K/V tiles a block in shared memory (three blocks an SM): the same results,
    alone and with the splits as a cluster or through scratch memory, at page edges and short contexts."""
    o = ops()
    dim, page = 128, 16
    lengths = [1, 63, 64, 65, 127, 129, 700, 1500, 16, 17]
    k_pool, v_pool, table, ks, vs = paged_setup(torch.bfloat16, lengths, kv_heads, dim, page, seed=splits)
    gen = torch.Generator().manual_seed(77)
    qs = [torch.randn(1, q_heads, dim, generator=gen).to(torch.bfloat16) for _ in lengths]
    q = torch.cat(qs).reshape(-1, q_heads * dim).cuda()
    cu = torch.arange(len(lengths) + 1, dtype=torch.int32, device="cuda")
    ctx = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    outs = []
    for stages in (2, 3):
        out = torch.full_like(q, float("nan"))
        o.attention_decode_bf16(q, k_pool, v_pool, out, table, cu, ctx, None, len(lengths), q_heads, kv_heads, dim, page,
                                1.0 / math.sqrt(dim), 0, splits, stages)
        outs.append(out)
    expected = []
    for s, n in enumerate(lengths):
        full_q = torch.zeros(n, q_heads, dim, dtype=torch.bfloat16)
        full_q[-1:] = qs[s]
        expected.append(plain_attention(full_q, ks[s], vs[s], None)[-1:])
    assert not torch.isnan(outs[0]).any()
    close(outs[0].cpu().view(-1, q_heads, dim), torch.cat(expected), torch.bfloat16)
    assert torch.equal(outs[0], outs[1])          # the same tiles in the same order: the same bits as three stages


@pytest.mark.parametrize("window", [1, 7, 64, 65, 300])
def test_attention_decode_bf16_window(window):
    lengths = [1, 50, 64, 65, 300, 777]
    got, expected, _, _ = run_attention(torch.bfloat16, lengths, [1] * 6, 4, 2, 32, 8, window=window, kernel="decode", splits=3)
    close(got, expected, torch.bfloat16)


@pytest.mark.parametrize("kernel", ["prefill", "decode"])
@pytest.mark.parametrize("far_key", [0, 15, 16, 63, 64, 65, 255, 256, 1023, 1024, 1500, 2046, 2047])
def test_bf16_attention_finds_one_far_key_among_thousands(kernel, far_key):
    dim, n = 128, 2048
    gen = torch.Generator().manual_seed(3)
    direction = torch.randn(dim, generator=gen)
    direction /= direction.norm()
    k_pool, v_pool, table, ks, vs = paged_setup(torch.bfloat16, [n], 1, dim, 16, seed=4)
    page = int(table[0, far_key // 16])
    k_pool[page, 0, far_key % 16] = (direction * 40.0).to(torch.bfloat16).cuda()
    v_pool[page, 0, far_key % 16] = 7.0
    o = ops()
    q = (direction * 40.0).to(torch.bfloat16).view(1, dim).cuda()
    out = torch.empty(1, dim, device="cuda", dtype=torch.bfloat16)
    one = torch.ones(1, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    if kernel == "prefill":
        o.attention_prefill_bf16(q, k_pool, v_pool, out, table, cu, n * one, 0 * one, 0 * one, 1, 1, 1, dim, 16, 1.0 / math.sqrt(dim))
    else:
        o.attention_decode_bf16(q, k_pool, v_pool, out, table, cu, n * one, None, 1, 1, 1, dim, 16, 1.0 / math.sqrt(dim), 0, 7)
    assert (out.float().cpu() - 7.0).abs().max() < 0.05


@pytest.mark.parametrize("tokens", [1, 3, 8, 16, 512, 700, 2048])
@pytest.mark.parametrize("q_heads, kv_heads, hidden", [(32, 8, 2560), (4, 2, 1024), (3, 1, 512), (16, 8, 1024)])
def test_fused_qkv_projection_equals_product_then_head_kernel(q_heads, kv_heads, hidden, tokens):
    """The q/k/v projection with norm, rotation and page write in its epilogue leaves the same bits in
    the query buffer and the pages as the product followed by the per-head kernel: the few-token
    kernel up to 16 tokens, pairs of blocks from 512 on (an odd number of heads leaves half a tile)."""
    o = ops()
    dim = 128
    page = {32: 16, 4: 32, 3: 8, 16: 64}[q_heads]           # pages of other sizes than the engine's usual 16 too
    pages = max(9, tokens // page + 3)
    gen = torch.Generator().manual_seed(tokens * 1000 + q_heads)
    rows = (q_heads + 2 * kv_heads) * dim
    h = torch.randn(tokens, hidden, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(rows, hidden, generator=gen) / math.sqrt(hidden)).to(torch.bfloat16).cuda()
    q_w = (1 + 0.2 * torch.randn(dim, generator=gen)).cuda()
    k_w = (1 + 0.2 * torch.randn(dim, generator=gen)).cuda()
    positions = torch.randint(0, 4000, (tokens,), generator=gen).to(torch.int32).cuda()
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, dim, 2).float() / dim))).cuda()
    table = torch.empty(tokens, 2, dim // 2, dtype=torch.float32, device="cuda")
    o.rope_table(positions, inv_freq, table)
    slots = torch.randperm(pages * page, generator=gen)[:tokens].to(torch.int32).cuda()

    def pools():
        return (torch.zeros(pages, kv_heads, page, dim, dtype=torch.bfloat16, device="cuda"),
                torch.zeros(pages, kv_heads, page, dim, dtype=torch.bfloat16, device="cuda"))

    k1, v1 = pools()
    qkv = torch.empty(tokens, rows, dtype=torch.bfloat16, device="cuda")
    o.gemm_tcgen05(h, w, qkv, max_splits=1 if tokens >= 512 else 0)     # the fused many-token product never splits K
    q1 = torch.empty(tokens, q_heads * dim, dtype=torch.bfloat16, device="cuda")
    o.qk_norm_rope_kv(qkv, q1, k1, v1, q_w, k_w, table, slots, q_heads, kv_heads, dim, page, 1e-6)
    k2, v2 = pools()
    q2 = torch.full_like(q1, float("nan"))
    for _ in range(2):
        taken = o.gemm_qkv_heads(h, w, q2, k2, v2, q_w, k_w, table, slots, q_heads, kv_heads, dim, page, 1e-6)
    assert o.gemm_status() == 0
    if not taken:
        # too few K blocks to split, nothing to split for, or clusters (pairs) switched off for the run
        if tokens >= 512:
            assert os.environ.get("LAYOVER_B200_GEMM_PAIR") == "0"
        else:
            assert hidden // 64 < 8 or rows // 128 >= 148 or os.environ.get("LAYOVER_B200_CLUSTER_REDUCE") == "0"
        return
    assert torch.equal(q1, q2)
    assert torch.equal(k1, k2) and torch.equal(v1, v2)


@pytest.mark.parametrize("m, inter, k", [(1, 64, 64), (8, 9728, 2560), (17, 128, 96), (64, 192, 200), (128, 1024, 256),
                                         (129, 64, 64), (300, 448, 136), (2048, 1280, 512), (2048, 9728, 256)])
def test_gemm_tcgen05_swiglu_epilogue(m, inter, k):
    o = ops()
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(inter, k, device="cuda") * 2 / math.sqrt(k)).to(torch.bfloat16)
    up = (torch.randn(inter, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
    w = o.interleave_gate_up(gate, up)
    assert w.shape == (2 * inter, k) and torch.equal(w[:64], gate[:64]) and torch.equal(w[64:128], up[:64])
    g = (a.double() @ gate.double().T).float().to(torch.bfloat16)
    u = (a.double() @ up.double().T).float().to(torch.bfloat16)
    expected = (torch.nn.functional.silu(g) * u).float()
    for _ in range(2):
        out = torch.full((m, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
        o.gemm_tcgen05(a, w, out, epilogue="swiglu")
        assert o.gemm_status() == 0
        assert not torch.isnan(out).any()
        close(out, expected, torch.bfloat16)
    with pytest.raises(ValueError, match="swiglu"):
        o.gemm_tcgen05(a, w[:2 * inter - 64], torch.empty(m, inter - 32, device="cuda", dtype=torch.bfloat16), epilogue="swiglu")


def run_tc_attention(lengths, q_lens, q_heads, kv_heads, page, window=0, seed=0, layers=3, layer=1):
    """The tcgen05 kernels against the plain attention: the pool has several layers and both planes,
    as the cache manager lays it out, and only plane (layer, K / V) holds the data."""
    o = ops()
    dim = 128
    k_pool, v_pool, table, ks, vs = paged_setup(torch.bfloat16, lengths, kv_heads, dim, page, seed)
    pages = k_pool.shape[0]
    pool = torch.full((layers, 2, pages, kv_heads, page, dim), float("nan"), dtype=torch.bfloat16, device="cuda")
    pool[layer, 0], pool[layer, 1] = k_pool, v_pool
    gen = torch.Generator().manual_seed(seed + 1)
    qs = [torch.randn(n, q_heads, dim, generator=gen).to(torch.bfloat16) for n in q_lens]
    q = torch.cat(qs).reshape(-1, q_heads * dim).cuda()
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device="cuda")
    ctx = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    scale = 1.0 / math.sqrt(dim)
    tiles = [(s, q0) for s, n in enumerate(q_lens) for q0 in range(0, n, 128)]
    tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
    tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
    o.attention_tcgen05_prefill(q, pool, layer, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads, kv_heads,
                                dim, page, scale, window)
    assert o.attention_tcgen05_status() == 0
    expected = []
    for s, n in enumerate(lengths):
        full_q = torch.zeros(n, q_heads, dim, dtype=torch.bfloat16)
        full_q[n - q_lens[s]:] = qs[s]
        expected.append(plain_attention(full_q, ks[s], vs[s], window or None)[n - q_lens[s]:])
    return out.cpu().view(-1, q_heads, dim), torch.cat(expected)


@pytest.mark.parametrize("q_heads, kv_heads, page", [(4, 1, 16), (2, 2, 8), (32, 8, 16), (3, 1, 32), (8, 2, 128)])
def test_attention_tcgen05_prefill(q_heads, kv_heads, page):
    lengths = [37, 300, 128, 129, 127, 1, 65, 256, 700]
    q_lens = [37, 129, 128, 1, 127, 1, 2, 256, 300]
    for _ in range(2):
        got, expected = run_tc_attention(lengths, q_lens, q_heads, kv_heads, page)
        assert not torch.isnan(got).any()              # NaN in unused slots, pages and planes did not leak
        close(got, expected, torch.bfloat16)


@pytest.mark.parametrize("window", [1, 5, 128, 200])
def test_attention_tcgen05_prefill_window(window):
    got, expected = run_tc_attention([270, 440, 33], [270, 3, 1], 4, 2, 16, window=window)
    close(got, expected, torch.bfloat16)


def tail_attention(q_tail, k, v, group):
    """Causal attention for the last rows of a sequence only (32-bit, on the CPU): q_tail [n, heads, dim]
    are the queries of the last n positions of keys k, v [len, kv_heads, dim]."""
    n, length = q_tail.shape[0], k.shape[0]
    kf = k.float().repeat_interleave(group, dim=1)
    vf = v.float().repeat_interleave(group, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q_tail.float(), kf) / math.sqrt(q_tail.shape[-1])
    position = torch.arange(length - n, length)[:, None]
    scores = scores.masked_fill(torch.arange(length)[None, :] > position, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), vf)


@pytest.mark.parametrize("kernel", ["tcgen05", "prefill", "decode", "decode16"])
def test_attention_over_long_contexts(kernel):
    """Contexts of some 20,000 keys: block tables wider than the slice that a block keeps in shared
    memory (1,024 pages), many tiles per block, and for decode many splits."""
    o = ops()
    dim, page, q_heads, kv_heads = 128, 16, 4, 1
    lengths = [20000, 17013]
    q_lens = [1, 1] if kernel.startswith("decode") else [200, 130]
    k_pool, v_pool, table, ks, vs = paged_setup(torch.bfloat16, lengths, kv_heads, dim, page, seed=3)
    gen = torch.Generator().manual_seed(4)
    qs = [torch.randn(n, q_heads, dim, generator=gen).to(torch.bfloat16) for n in q_lens]
    q = torch.cat(qs).reshape(-1, q_heads * dim).cuda()
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device="cuda")
    ctx = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    scale = 1.0 / math.sqrt(dim)
    if kernel.startswith("decode"):
        splits = 16 if kernel == "decode16" else o.decode_splits(2, q_heads, kv_heads, dim, max(lengths), 148)
        o.attention_decode_bf16(q, k_pool, v_pool, out, table, cu, ctx, None, 2, q_heads, kv_heads, dim, page, scale, 0, splits)
    else:
        size = 128 if kernel == "tcgen05" else o.attention_mma_block_queries()
        tiles = [(s, q0) for s, n in enumerate(q_lens) for q0 in range(0, n, size)]
        tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
        tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
        if kernel == "tcgen05":
            pool = torch.stack((k_pool, v_pool))[None].contiguous()
            o.attention_tcgen05_prefill(q, pool, 0, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads, kv_heads,
                                        dim, page, scale, 0)
            assert o.attention_tcgen05_status() == 0
        else:
            o.attention_prefill_bf16(q, k_pool, v_pool, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads,
                                     kv_heads, dim, page, scale, 0)
    expected = torch.cat([tail_attention(qs[s], ks[s], vs[s], q_heads // kv_heads) for s in range(2)])
    assert not torch.isnan(out).any()
    close(out.cpu().view(-1, q_heads, dim), expected, torch.bfloat16)


@pytest.mark.parametrize("heads", [1, 2])
def test_attention_tcgen05_scores_far_apart_force_rescaling(heads):
    """Keys whose scores grow along the sequence make the running maximum jump by far more than the
    2^8 that the kernel tolerates before it rescales its accumulated output. One head goes through
    the kernel with a head per block, two through the one with two heads per block."""
    o = ops()
    dim, n, page = 128, 640, 16
    gen = torch.Generator().manual_seed(9)
    direction = torch.randn(dim, generator=gen)
    direction /= direction.norm()
    k_pool, v_pool, table, ks, vs = paged_setup(torch.bfloat16, [n], 1, dim, page, seed=5, poison=False)
    for key in range(n):                                       # key j scores about j / 8 in natural units
        k = (direction * (key / 8.0) * math.sqrt(dim) / 10.0).to(torch.bfloat16)
        k_pool[int(table[0, key // page]), 0, key % page] = k.cuda()
        ks[0][key, 0] = k
    q = (direction * 10.0).to(torch.bfloat16).view(1, 1, dim).repeat(n, heads, 1)
    q[:, -1] *= 0.5                                            # the heads differ
    pool = torch.stack((k_pool, v_pool))[None].contiguous()
    qf = q.reshape(n, heads * dim).cuda()
    out = torch.empty_like(qf)
    cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
    ctx = torch.tensor([n], dtype=torch.int32, device="cuda")
    tiles = list(range(0, n, 128))
    o.attention_tcgen05_prefill(qf, pool, 0, out, table, cu, ctx, torch.zeros(len(tiles), dtype=torch.int32, device="cuda"),
                                torch.tensor(tiles, dtype=torch.int32, device="cuda"), len(tiles), heads, 1, dim, page, 1 / math.sqrt(dim))
    assert o.attention_tcgen05_status() == 0
    expected = plain_attention(q, ks[0], vs[0])
    close(out.cpu().view(n, heads, dim), expected, torch.bfloat16)


@pytest.mark.parametrize("kernel", ["simt", "prefill", "decode", "tcgen05"])
def test_pools_of_more_than_2_to_the_31_elements(kernel):
    """Pages whose element offset does not fit 32 bits (the reference pins the same for its decode
    kernel, tests/test_triton_decode.py:277-300 there): the page-write kernel puts keys and values
    there and each attention kernel reads them back."""
    o = ops()
    q_heads, kv_heads, dim, page = 32, 8, 128, 16
    dtype = torch.float32 if kernel == "simt" else torch.bfloat16
    pages = (1 << 31) // (kv_heads * page * dim) + 40
    pool = torch.empty((1, 2, pages + 1, kv_heads, page, dim), dtype=dtype, device="cuda")
    k_pool, v_pool = pool[0, 0], pool[0, 1]
    assert k_pool.numel() > 2 ** 31
    lengths, q_lens = [70, 33, 130], ([70, 5, 128] if kernel != "decode" else [1, 1, 1])
    gen = torch.Generator().manual_seed(5)
    mine, at = [], pages                                  # the sequences' pages are the pool's last ones
    for n in lengths:
        count = -(-n // page)
        at -= count
        mine.append(list(range(at, at + count)))
    assert at * kv_heads * page * dim > 2 ** 31
    width = max(len(m) for m in mine)
    table = torch.full((len(lengths), width), pages, dtype=torch.int32)
    ks, vs, slots = [], [], []
    for s, n in enumerate(lengths):
        table[s, :len(mine[s])] = torch.tensor(mine[s], dtype=torch.int32)
        ks.append(torch.randn(n, kv_heads, dim, generator=gen).to(dtype))
        vs.append(torch.randn(n, kv_heads, dim, generator=gen).to(dtype))
        slots += [mine[s][pos // page] * page + pos % page for pos in range(n)]
    # the write: rows of [q | k | v] without norm or rotation
    total = sum(lengths)
    rows = torch.cat([torch.zeros(total, q_heads * dim, dtype=dtype), torch.cat(ks).reshape(total, -1),
                      torch.cat(vs).reshape(total, -1)], dim=1).cuda()
    pool[:, :, at:].fill_(float("nan"))
    o.qk_norm_rope_kv(rows, None, k_pool, v_pool, None, None, None, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                      q_heads, kv_heads, dim, page, 0.0)
    last = mine[2][-1]
    assert torch.equal(k_pool[last, :, (130 - 1) % page].cpu(), ks[2][-1]) and torch.equal(v_pool[mine[0][0], :, 0].cpu(), vs[0][0])
    qs = [torch.randn(n, q_heads, dim, generator=gen).to(dtype) for n in q_lens]
    q = torch.cat(qs).reshape(-1, q_heads * dim).cuda()
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device="cuda")
    ctx = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    bq = {"simt": o.attention_simt_block_queries, "prefill": o.attention_mma_block_queries,
          "decode": o.attention_mma_block_queries, "tcgen05": lambda: o.TCGEN05_TILE}[kernel]()
    tiles = [(s, q0) for s, n in enumerate(q_lens) for q0 in range(0, n, bq)]
    tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
    tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    scale, table = 1.0 / math.sqrt(dim), table.cuda()
    if kernel == "simt":
        o.attention_simt(q, k_pool, v_pool, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads, kv_heads, dim, page, scale)
    elif kernel == "prefill":
        o.attention_prefill_bf16(q, k_pool, v_pool, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads, kv_heads, dim,
                                 page, scale)
    elif kernel == "decode":
        o.attention_decode_bf16(q, k_pool, v_pool, out, table, cu, ctx, None, len(lengths), q_heads, kv_heads, dim, page, scale,
                                0, 2)
    else:
        o.attention_tcgen05_prefill(q, pool, 0, out, table, cu, ctx, tile_seq, tile_q0, len(tiles), q_heads, kv_heads, dim,
                                    page, scale)
        assert o.attention_tcgen05_status() == 0
    expected = []
    for s, n in enumerate(lengths):
        full_q = torch.zeros(n, q_heads, dim, dtype=dtype)
        full_q[n - q_lens[s]:] = qs[s]
        expected.append(plain_attention(full_q, ks[s], vs[s], None)[n - q_lens[s]:])
    got = out.cpu().view(-1, q_heads, dim)
    assert not torch.isnan(got).any()
    close(got, torch.cat(expected), dtype)
    del pool, k_pool, v_pool
    torch.cuda.empty_cache()


def test_decode_attention_gives_zeros_for_a_sequence_without_keys():
    """A length of 0 is not something the engine produces, but the exported C entry points take raw
    arrays from any caller: such a row gets zeros, not NaN, beside normal rows."""
    o = ops()
    q_heads, kv_heads, dim, page = 8, 2, 128, 16
    k_pool, v_pool, table, ks, vs = paged_setup(torch.bfloat16, [40, 1, 200], kv_heads, dim, page)
    ctx = torch.tensor([40, 0, 200], dtype=torch.int32, device="cuda")
    q = torch.randn(3, q_heads * dim).to(torch.bfloat16).cuda()
    cu = torch.arange(4, dtype=torch.int32, device="cuda")
    for splits in (1, 2, 3):
        out = torch.full_like(q, float("nan"))
        o.attention_decode_bf16(q, k_pool, v_pool, out, table, cu, ctx, None, 3, q_heads, kv_heads, dim, page,
                                1.0 / math.sqrt(dim), 0, splits)
        assert torch.equal(out[1], torch.zeros_like(out[1])) and not torch.isnan(out).any()
        full_q = torch.zeros(40, q_heads, dim, dtype=torch.bfloat16)
        full_q[-1] = q[0].cpu().view(q_heads, dim)
        close(out[0].cpu().view(q_heads, dim), plain_attention(full_q, ks[0], vs[0], None)[-1], torch.bfloat16)
