"""The allocation-free decode attention, called through its exported C symbol.

Some hosts hand the whole device to their own memory arena, or forbid allocator calls once a
latency-critical loop is warm; they cannot let a library allocate split-K scratch for them. For
them the library exports `lb_attention_decode_bf16_static`, whose scratch is a static device array
inside the library (csrc/decode_attention_static.h). This test calls that symbol directly with raw
pointers, twice in a row on different inputs (the second call finds the array as the first left
it), and checks each result against a plain 32-bit attention and against the regular entry point,
which takes caller-made scratch. That the call allocates nothing is checked where an allocation
would show: in the driver's count of free device memory, not in torch's own allocator.

The file sorts last so that a run which stops at the first failure has run everything else.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def static_entry():
    from layover_b200.csrc import build

    lib = build.load("decode_attention_static")
    fn = lib.lb_attention_decode_bf16_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] + [ctypes.c_void_p] * 2 + [ctypes.c_int] * 5 + \
                  [ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.lb_attention_decode_static_strerror.restype = ctypes.c_char_p
    lib.lb_attention_decode_static_strerror.argtypes = [ctypes.c_int]
    return fn, lib.lb_attention_decode_static_strerror


def make_case(seed, lengths, q_heads, kv_heads, dim, page):
    gen = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page) for n in lengths]
    total = sum(pages_per) + 1
    k_host = torch.randn(total, kv_heads, page, dim, generator=gen).to(torch.bfloat16)
    v_host = torch.randn(total, kv_heads, page, dim, generator=gen).to(torch.bfloat16)
    order = torch.randperm(total - 1, generator=gen).tolist()
    table = torch.full((len(lengths), max(pages_per)), total - 1, dtype=torch.int32)
    for s, count in enumerate(pages_per):
        table[s, :count] = torch.tensor([order.pop() for _ in range(count)], dtype=torch.int32)
    q = torch.randn(len(lengths), q_heads * dim, generator=gen).to(torch.bfloat16).cuda()
    cu = torch.arange(len(lengths) + 1, dtype=torch.int32).cuda()
    ctx = torch.tensor(lengths, dtype=torch.int32).cuda()
    return q, k_host.cuda(), v_host.cuda(), table.cuda(), cu, ctx


def plain_result(q, k_pool, v_pool, table, ctx, q_heads, kv_heads, dim, page):
    """The attention of each sequence's single query over its own keys, by the plain implementation."""
    from plain_qwen3 import plain_attention

    rows = []
    k_host, v_host, table = k_pool.cpu(), v_pool.cpu(), table.cpu()
    for s, n in enumerate(ctx.tolist()):
        pages = table[s, : -(-n // page)].long()
        keys = k_host[pages].permute(0, 2, 1, 3).reshape(-1, kv_heads, dim)[:n]        # [n, kv_heads, dim]
        values = v_host[pages].permute(0, 2, 1, 3).reshape(-1, kv_heads, dim)[:n]
        queries = torch.zeros(n, q_heads, dim, dtype=torch.bfloat16)
        queries[-1] = q[s].cpu().view(q_heads, dim)
        rows.append(plain_attention(queries, keys, values, None)[-1].reshape(-1))
    return torch.stack(rows)


def call_static(fn, q, k_pool, v_pool, table, cu, ctx, q_heads, kv_heads, dim, page, splits):
    import gc

    out = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    gc.collect()                                        # tensors that earlier tests left in cycles go now, not during the call
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]          # the driver's count: sees any cudaMalloc, whoever makes it
    asked = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
    code = call_symbol(fn, q, k_pool, v_pool, out, table, cu, ctx, q_heads, kv_heads, dim, page, splits, stream)
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == asked   # nothing asked of torch's allocator
    assert torch.cuda.mem_get_info()[0] >= free_before  # and nothing taken from the device behind its back
    return code, out


def call_symbol(fn, q, k_pool, v_pool, out, table, cu, ctx, q_heads, kv_heads, dim, page, splits, stream):
    return fn(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
              cu.data_ptr(), ctx.data_ptr(), ctx.shape[0], q_heads, kv_heads, dim, page, 1.0 / math.sqrt(dim), 0, splits,
              stream)


def test_static_scratch_entry_matches_the_regular_one_on_two_calls_in_a_row():
    from layover_b200 import ops

    fn, strerror = static_entry()
    q_heads, kv_heads, dim, page = 32, 8, 128, 16
    warm = make_case(1, [40, 300], q_heads, kv_heads, dim, page)
    # the first call on a device looks up the array's address and loads the kernels (a module load may
    # take device memory once); the calls that are measured come after it
    assert call_symbol(fn, *warm[:3], torch.empty_like(warm[0]), *warm[3:], q_heads, kv_heads, dim, page, 3,
                       torch.cuda.current_stream().cuda_stream) == 0
    ops.attention_decode_bf16(warm[0], warm[1], warm[2], torch.empty_like(warm[0]), warm[3], warm[4], warm[5], None, 2,
                              q_heads, kv_heads, dim, page, 1.0 / math.sqrt(dim), 0, 3)
    torch.cuda.synchronize()
    # 5 and 7 splits: both entries merge through scratch memory, the same bits; 4 splits: the regular entry
    # merges inside a cluster in another order, equal within rounding
    for call, (lengths, splits) in enumerate((([700, 1, 64, 1000, 257], 5), ([129, 2048, 33], 7), ([600, 90, 1500], 4))):
        case = make_case(10 + call, lengths, q_heads, kv_heads, dim, page)
        q, k_pool, v_pool, table, cu, ctx = case
        code, got = call_static(fn, *case, q_heads, kv_heads, dim, page, splits)
        assert code == 0, strerror(code).decode()
        regular = torch.empty_like(q)
        ops.attention_decode_bf16(q, k_pool, v_pool, regular, table, cu, ctx, None, len(lengths), q_heads, kv_heads, dim,
                                  page, 1.0 / math.sqrt(dim), 0, splits)
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        expected = plain_result(q, k_pool, v_pool, table, ctx, q_heads, kv_heads, dim, page)
        # the tolerance of the other attention tests: 4 * 2^-7 * max|reference|
        bound = 4 * 2.0 ** -7 * expected.float().abs().max().item()
        assert (got.float().cpu() - expected.float()).abs().max().item() <= bound
        assert (got.float() - regular.float()).abs().max().item() <= bound
        if splits != 4:
            assert torch.equal(got, regular)   # the same kernel and the same split order: the same bits


def test_static_scratch_entry_refuses_what_does_not_fit():
    fn, strerror = static_entry()
    case = make_case(3, [40] * 600, 32, 8, 128, 16)               # 4800 (sequence, KV head) counters > 4096
    code, _ = call_static(fn, *case, 32, 8, 128, 16, 2)
    assert code == -20 and b"static array" in strerror(code)
    case = make_case(4, [500] * 64, 32, 8, 128, 16)               # 64 * 32 * 8 * 130 partial floats > 1 Mi
    code, _ = call_static(fn, *case, 32, 8, 128, 16, 8)
    assert code == -20
    code, out = call_static(fn, *case, 32, 8, 128, 16, 1)         # unsplit needs no scratch at all
    torch.cuda.synchronize()
    assert code == 0 and not torch.isnan(out).any()
    code, _ = call_static(fn, *make_case(5, [10], 34, 2, 128, 16), 34, 2, 128, 16, 2)   # 17 heads per KV head
    assert code == -22
