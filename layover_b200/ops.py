"""The engine's device operations: thin, checked wrappers over the CUDA kernels of `csrc/`.

Every function takes CUDA tensors, launches on torch's current stream and returns without
synchronising. There is no other implementation behind them: if the kernels cannot be
compiled or loaded, or a tensor is not on a CUDA device, the call raises. A size or alignment
that a kernel does not support is refused with a ValueError before or by the launch.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from .csrc import build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_REFUSALS = {-1: "unsupported dtype", -2: "unsupported size", -3: "unsupported alignment"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}; the engine runs float32 or bfloat16") from None


LAUNCHES = 0   # kernels of this package launched (or captured into a graph) so far


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code in _REFUSALS:
        raise ValueError(f"{what}: {_REFUSALS[code]}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("layover_b200 kernels need CUDA tensors: there is no CPU path")
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


_signatures_done: set[str] = set()


def _fn(lib_name: str, fn_name: str, argtypes):
    lib = build.load(lib_name)
    fn = getattr(lib, fn_name)
    key = lib_name + "." + fn_name
    if key not in _signatures_done:
        fn.argtypes = argtypes
        fn.restype = c_int
        _signatures_done.add(key)
    return fn


# ------------------------------------------------------------------ elementwise
RECORD_WORDS = 8                 # int32 words of a request's record on the device (csrc/common.cuh)
RECORD_POSITION, RECORD_SEED_LO, RECORD_SEED_HI, RECORD_COUNT, RECORD_TEMPERATURE, RECORD_LAST_TOKEN = range(6)


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, token_src: torch.Tensor | None = None,
          records: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[id]; ids int32 [T], table [V, H], out [T, H]. Where token_src[t] >= 0 the id is the
    last token in row token_src[t] of `records` (int32 [slots, RECORD_WORDS]) instead of ids[t]."""
    _need(ids, torch.int32, "ids"); _need(table, None, "table"); _need(out, table.dtype, "out")
    if (token_src is None) != (records is None):
        raise ValueError("embed: token_src and records come together")
    if token_src is not None:
        _need(token_src, torch.int32, "token_src"); _need(records, torch.int32, "records")
        if records.dim() != 2 or records.shape[1] != RECORD_WORDS or token_src.shape[0] != ids.shape[0]:
            raise ValueError("embed: records must be [slots, RECORD_WORDS] and token_src one entry per token")
    fn = _fn("elementwise", "lb_embed", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(table.dtype), _ptr(ids), _ptr(token_src), _ptr(records), _ptr(table), _ptr(out), ids.shape[0],
              table.shape[1], table.shape[0], _stream()), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """x += delta (in place, unless `rows` picks source rows), out = rmsnorm(x) * weight.

    x, delta [T, H]; weight float32 [H]; out [T or len(rows), H]."""
    _need(x, None, "x"); _need(weight, torch.float32, "weight"); _need(out, x.dtype, "out")
    if delta is not None:
        _need(delta, x.dtype, "delta")
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if out.shape[0] < n_rows or out.shape[-1] != x.shape[-1] or weight.shape[0] != x.shape[-1]:
        raise ValueError("add_rmsnorm: shapes do not agree")
    fn = _fn("elementwise", "lb_add_rmsnorm",
             [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(dtype_code(x.dtype), _ptr(x), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_rows, x.shape[-1],
              float(eps), _stream()), "add_rmsnorm")
    return out


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, 0, i] = cos(positions[t] * inv_freq[i]), out[t, 1, i] = sin(...); out float32 [T, 2, n_freq]."""
    _need(positions, torch.int32, "positions"); _need(inv_freq, torch.float32, "inv_freq"); _need(out, torch.float32, "out")
    tokens, n_freq = positions.shape[0], inv_freq.shape[0]
    if tuple(out.shape) != (tokens, 2, n_freq):
        raise ValueError("rope_table: out must be [tokens, 2, n_freq]")
    fn = _fn("elementwise", "lb_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(positions), _ptr(inv_freq), _ptr(out), tokens, n_freq, _stream()), "rope_table")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, q_out: torch.Tensor | None, k_pool: torch.Tensor | None,
                    v_pool: torch.Tensor | None, q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None,
                    table: torch.Tensor | None, slot_map: torch.Tensor | None, q_heads: int, kv_heads: int, dim: int,
                    page_tokens: int, eps: float) -> None:
    """Per-head norm and rotation of q and k in a fused projection row, q to q_out, k and v to their pages.

    qkv [T, (q_heads + 2 kv_heads) * dim]; q_out [T, q_heads * dim]; pools [pages, kv_heads, page_tokens, dim];
    table float32 [T, 2, dim / 2] from `rope_table` (None: no rotation)."""
    tokens = qkv.shape[0]
    _need(qkv, None, "qkv")
    if q_out is not None:
        _need(q_out, qkv.dtype, "q_out")
    if qkv.shape[1] != (q_heads + 2 * kv_heads) * dim:
        raise ValueError("qk_norm_rope_kv: projection row does not match the head counts")
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        if t is not None:
            _need(t, torch.float32, name)
    if table is not None and (table.dim() != 3 or table.shape[0] != tokens or table.shape[1] != 2):
        raise ValueError("qk_norm_rope_kv: the rotary table must be [tokens, 2, n_freq]")
    if k_pool is not None:
        _need(k_pool, qkv.dtype, "k_pool"); _need(v_pool, qkv.dtype, "v_pool"); _need(slot_map, torch.int32, "slot_map")
    n_freq = 0 if table is None else table.shape[2]
    fn = _fn("elementwise", "lb_qk_norm_rope_kv",
             [c_int] + [c_void_p] * 8 + [c_int] * 6 + [c_float, c_void_p])
    _check(fn(dtype_code(qkv.dtype), _ptr(qkv), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_norm_w),
              _ptr(k_norm_w), _ptr(table), _ptr(slot_map), tokens, q_heads, kv_heads, dim, n_freq,
              page_tokens, float(eps), _stream()), "qk_norm_rope_kv")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> torch.Tensor:
    """out = silu(gate) * up, gate_up [T, 2 I], out [T, I]. block 0: the row is [all gates | all ups];
    block b: gates and ups alternate in blocks of b features (`interleave_gate_up`'s layout)."""
    _need(gate_up, None, "gate_up"); _need(out, gate_up.dtype, "out")
    inter = gate_up.shape[1] // 2
    if gate_up.shape[1] != 2 * inter or out.shape[1] != inter or out.shape[0] != gate_up.shape[0]:
        raise ValueError("swiglu: shapes do not agree")
    fn = _fn("elementwise", "lb_swiglu", [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(dtype_code(gate_up.dtype), _ptr(gate_up), _ptr(out), gate_up.shape[0], inter, int(block), _stream()),
           "swiglu")
    return out


# ------------------------------------------------------------------ matrix products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit FFMA accumulation (no tensor cores).

    a and w share a dtype (float32 or bfloat16); out has it too, or float32. Rows may be strided."""
    if a.dtype != w.dtype or a.dim() != 2 or w.dim() != 2 or out.dim() != 2:
        raise ValueError("gemm: operands must be 2-D and share a dtype")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise ValueError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("gemm: innermost dimension must be contiguous")
    fn = _fn("gemm_simt", "lb_gemm_simt",
             [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long, c_void_p])
    _check(fn(dtype_code(a.dtype), dtype_code(out.dtype), _ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0),
              w.stride(0), out.stride(0), _stream()), "gemm_simt")
    return out


# ------------------------------------------------------------------ attention
def attention_simt_block_queries() -> int:
    lib = build.load("attention_simt")
    lib.lb_attention_simt_block_queries.restype = c_int
    return lib.lb_attention_simt_block_queries()


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                   block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, tile_seq: torch.Tensor,
                   tile_q0: torch.Tensor, n_tiles: int, q_heads: int, kv_heads: int, dim: int, page_tokens: int,
                   scale: float, window: int = 0) -> torch.Tensor:
    """Paged causal attention in 32-bit arithmetic for any mix of segment lengths.

    q, out [T, q_heads * dim]; pools [pages, kv_heads, page_tokens, dim]; block_table int32 [S, W];
    cu_q int32 [S + 1]; ctx_len int32 [S]; (tile_seq, tile_q0) int32 [n_tiles] list the query tiles."""
    _need(q, None, "q"); _need(out, q.dtype, "out"); _need(k_pool, q.dtype, "k_pool"); _need(v_pool, q.dtype, "v_pool")
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _need(t, torch.int32, name)
    fn = _fn("attention_simt", "lb_attention_simt",
             [c_int] + [c_void_p] * 5 + [c_int] + [c_void_p] * 4 + [c_int] * 5 + [c_float, c_int, c_void_p])
    _check(fn(dtype_code(q.dtype), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table),
              block_table.shape[1], _ptr(cu_q), _ptr(ctx_len), _ptr(tile_seq), _ptr(tile_q0), n_tiles, q_heads,
              kv_heads, dim, page_tokens, float(scale), int(window), _stream()), "attention_simt")
    return out


def attention_f32(q, cache, out, block_table, batch, q_heads, kv_heads, dim, page_tokens, scale, window):
    """The 32-bit path's attention for one step: one kernel for every mix of segment lengths."""
    tiles = batch.tiles[attention_simt_block_queries()]
    attention_simt(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, tiles.tile_seq, tiles.tile_q0,
                   tiles.count, q_heads, kv_heads, dim, page_tokens, scale, window)


# ------------------------------------------------------------------ sampling
def sample(logits: torch.Tensor, tokens: torch.Tensor, records: torch.Tensor | None = None,
           row_slots: torch.Tensor | None = None, positions: torch.Tensor | None = None,
           logit_rows: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """tokens[r] = the next token of row r of logits (float32 [R, V], rows may be strided).

    With `records` (int32 [slots, RECORD_WORDS]) and `row_slots` (int32 [R]) row r belongs to the
    request in slot row_slots[r]: temperature 0 there is the first index of the maximum, otherwise a
    Gumbel-max draw keyed by the record's seed and counter; the kernel stores the token as the
    record's last token, bumps its counter and, given `positions` [T] and `logit_rows` [R], sets its
    position. Without records every row is greedy. `status` (int64 device addresses of other
    libraries' error words, from `status_words`) are copied to tokens[R:], so tokens holds
    R + len(status) ints."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("sample: logits must be float32 [rows, vocab] with a contiguous vocabulary")
    _need(tokens, torch.int32, "tokens")
    rows, vocab = logits.shape
    n_status = 0 if status is None else status.shape[0]
    if tokens.shape[0] < rows + n_status:
        raise ValueError("sample: tokens must hold a word per row and per status word")
    if records is not None:
        _need(records, torch.int32, "records"); _need(row_slots, torch.int32, "row_slots")
        if records.dim() != 2 or records.shape[1] != RECORD_WORDS or row_slots.shape[0] < rows:
            raise ValueError("sample: records must be [slots, RECORD_WORDS] and row_slots one entry per row")
    for name, t in (("positions", positions), ("logit_rows", logit_rows)):
        if t is not None:
            _need(t, torch.int32, name)
    if status is not None:
        _need(status, torch.int64, "status")
    fn = _fn("sampling", "lb_sample", [c_void_p, c_long, c_int, c_int] + [c_void_p] * 6 + [c_int, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), rows, vocab, _ptr(records), _ptr(row_slots), _ptr(positions),
              _ptr(logit_rows), _ptr(tokens), _ptr(status), n_status, _stream()), "sample")
    return tokens


# ------------------------------------------------------------------ error words of the tensor-core kernels
# Every wait inside the tcgen05 kernels is bounded; a wait that runs out records a code in the
# library's error word and the block leaves. The sampling kernel copies those words behind the
# tokens it writes, so the host sees them with every step's tokens and without a synchronisation
# of its own (`Sampler`); `status_words` lists them, `explain_status` names a code's library, and
# `reset_after_error` puts back what such a block may have left behind (counters that a launch
# normally returns to zero).
_STATUS_LIBRARIES = (("gemm_tcgen05", "lb_gemm_tcgen05_status_address", "lb_gemm_tcgen05_status"),
                     ("attention_tcgen05", "lb_attention_tcgen05_status_address", "lb_attention_tcgen05_status"))
_status_words: dict[tuple[int, tuple[str, ...]], tuple[torch.Tensor, tuple[str, ...]]] = {}


def status_words(device: torch.device, libraries) -> tuple[torch.Tensor | None, tuple[str, ...]]:
    """(int64 device tensor of the error words' addresses, the libraries they belong to) for those of
    `libraries` that have one; (None, ()) if none has."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    wanted = tuple(name for name, _, _ in _STATUS_LIBRARIES if name in libraries)
    key = (index, wanted)
    if key not in _status_words:
        addresses = []
        with torch.cuda.device(index):
            for name, getter, _ in _STATUS_LIBRARIES:
                if name in wanted:
                    fn = getattr(build.load(name), getter)
                    fn.restype = c_void_p
                    address = fn()
                    if not address:
                        raise KernelError(f"{name}: the address of its error word cannot be had")
                    addresses.append(address)
            tensor = torch.tensor(addresses, dtype=torch.int64, device="cuda") if addresses else None
        _status_words[key] = (tensor, wanted)
    return _status_words[key]


def reset_after_error(device: torch.device) -> None:
    """After a kernel reported a wait that ran out: wait for the device, clear the error words and zero
    the split counters (a block that gave up does not take part in returning them to zero)."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    with torch.cuda.device(index):
        torch.cuda.synchronize()
        for name, _, clear in _STATUS_LIBRARIES:
            if name in build.loaded():
                fn = getattr(build.load(name), clear)
                fn.restype = c_int
                fn()
        if index in _scratch:
            _scratch[index][1].zero_()
        if index in _attn_scratch:
            _attn_scratch[index][1].zero_()
        torch.cuda.synchronize()


# ------------------------------------------------------------------ the bfloat16 path
# Split-K scratch and counters are one set per device, shared by every model, engine and stream of
# the process: a launch leaves its counters at zero for the next one, and two launches that overlap
# on the device would mix their partial tiles. So all launches of a device must be ordered on ONE
# stream (the engine runs everything on torch's current stream; the warm-up of a graph capture runs
# on a side stream only while the main stream waits for it).
_SCRATCH_FLOATS = 8 << 20     # split-K partial tiles (32 MiB)
_SCRATCH_COUNTERS = 4096
_scratch: dict[int, tuple[torch.Tensor, torch.Tensor, int]] = {}


def gemm_scratch(device: torch.device) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Per device: the split-K scratch, its tile counters (zero between launches) and the SM count.
    Made once, outside any graph capture (models call this when their runtime is made)."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    if index not in _scratch:
        with torch.cuda.device(index):
            partials = torch.empty(_SCRATCH_FLOATS, dtype=torch.float32, device="cuda")
            counters = torch.zeros(_SCRATCH_COUNTERS, dtype=torch.int32, device="cuda")
        _scratch[index] = (partials, counters, torch.cuda.get_device_properties(index).multi_processor_count)
    return _scratch[index]


def gemm_tcgen05_supports(a: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides: K-contiguous rows whose stride is a multiple of 8."""
    return (a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1)


SWIGLU_BLOCK = 64   # gate and up rows alternate in blocks of this many features for the fused epilogue


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2 I, H] with rows in blocks of 64 gate rows followed by the 64 up rows of the same features:
    the layout `gemm_tcgen05(..., epilogue="swiglu")` wants. I must be a multiple of 64."""
    inter, hidden = gate.shape
    if inter % SWIGLU_BLOCK or up.shape != gate.shape:
        raise ValueError("interleave_gate_up: the width must be a multiple of 64 and the shapes must agree")
    blocks = inter // SWIGLU_BLOCK
    stacked = torch.stack((gate.view(blocks, SWIGLU_BLOCK, hidden), up.view(blocks, SWIGLU_BLOCK, hidden)), dim=1)
    return stacked.reshape(2 * inter, hidden).contiguous()


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, max_splits: int = 0,
                 epilogue: str | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores; bfloat16 in, out bfloat16 or float32.

    epilogue "swiglu": w's rows are interleaved by `interleave_gate_up` and out[M, N / 2] = silu(gate) * up,
    rounded where the reference's bfloat16 tensors round."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        raise ValueError("gemm_tcgen05: operands must be 2-D bfloat16")
    m, k = a.shape
    n = w.shape[0]
    if epilogue not in (None, "swiglu"):
        raise ValueError(f"gemm_tcgen05: unknown epilogue {epilogue!r}")
    out_cols = n // 2 if epilogue == "swiglu" else n
    if epilogue == "swiglu" and (n % (2 * SWIGLU_BLOCK) or out.dtype != torch.bfloat16):
        raise ValueError("gemm_tcgen05: the swiglu epilogue needs interleaved weights (2 I rows, I % 64 == 0) and a bfloat16 output")
    if w.shape[1] != k or tuple(out.shape) != (m, out_cols) or out.stride(1) != 1:
        raise ValueError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    partials, counters, sms = gemm_scratch(a.device)
    fn = _fn("gemm_tcgen05", "lb_gemm_tcgen05",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_long, c_long, c_long, c_void_p, c_long,
              c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0), out.stride(0),
              _ptr(partials), partials.numel(), _ptr(counters), counters.numel(), sms, int(max_splits),
              1 if epilogue == "swiglu" else 0, _stream()), "gemm_tcgen05")
    return out


def gemm_qkv_heads(h: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   q_norm_w: torch.Tensor, k_norm_w: torch.Tensor, table: torch.Tensor, slot_map: torch.Tensor,
                   q_heads: int, kv_heads: int, dim: int, page_tokens: int, eps: float) -> bool:
    """The stacked q/k/v projection of up to 16 tokens, or of 512 and more, with the per-head norm, the
    rotation and the page write in its epilogue (head size 128): leaves in q_out and the pools what
    `gemm_tcgen05` followed by `qk_norm_rope_kv` leaves there, bit for bit. False: these sizes are not
    taken and nothing was launched."""
    tokens = h.shape[0]
    if (dim != 128 or 16 < tokens < 512 or h.dtype != torch.bfloat16 or q_norm_w is None or k_norm_w is None or table is None
            or k_pool is None or not gemm_tcgen05_supports(h, w_qkv)):
        return False
    for name, t in (("h", h), ("w_qkv", w_qkv), ("q_out", q_out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        _need(t, torch.float32, name)
    _need(slot_map, torch.int32, "slot_map")
    if w_qkv.shape != ((q_heads + 2 * kv_heads) * dim, h.shape[1]) or tuple(table.shape) != (tokens, 2, dim // 2) \
            or q_out.shape != (tokens, q_heads * dim) or not q_out.is_contiguous():
        raise ValueError("gemm_qkv_heads: shapes do not agree")
    sms = gemm_scratch(h.device)[2]
    fn = _fn("gemm_tcgen05", "lb_gemm_qkv_heads",
             [c_void_p, c_void_p, c_int, c_int, c_long, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p])
    code = fn(_ptr(h), _ptr(w_qkv), tokens, h.shape[1], h.stride(0), w_qkv.stride(0), q_heads, kv_heads, dim,
              _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table), table.shape[2], _ptr(slot_map), _ptr(q_out), _ptr(k_pool),
              _ptr(v_pool), page_tokens, float(eps), sms, _stream())
    if code == 1:
        return False
    _check(code, "gemm_qkv_heads")
    return True


def gemm_status() -> int:
    """0, or the code a tensor-core product recorded when one of its bounded waits ran out
    (1 loads, 2 MMAs, 3 epilogue). Synchronises; clears the code."""
    lib = build.load("gemm_tcgen05")
    lib.lb_gemm_tcgen05_status.restype = c_int
    torch.cuda.synchronize()
    return lib.lb_gemm_tcgen05_status()


def gemm_set_status(code: int) -> None:
    """Write the tensor-core product's error word from the host (a drill of the reporting path)."""
    lib = build.load("gemm_tcgen05")
    lib.lb_gemm_tcgen05_set_status.restype = c_int
    lib.lb_gemm_tcgen05_set_status.argtypes = [c_int]
    torch.cuda.synchronize()
    if lib.lb_gemm_tcgen05_set_status(int(code)):
        raise KernelError("gemm_tcgen05: cannot write the error word")


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T, bfloat16 operands, 32-bit accumulation; out bfloat16 or float32.
    Shapes that TMA cannot address (a row stride that is no multiple of 16 bytes) take the FFMA kernel."""
    if gemm_tcgen05_supports(a, w):
        return gemm_tcgen05(a, w, out)
    return gemm_simt(a, w, out)


_attn_scratch: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
_ATTN_SCRATCH_FLOATS = 8 << 20     # split-K partial outputs (32 MiB)
_ATTN_COUNTERS = 1 << 16


def attention_scratch(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Per device: scratch for the decode kernel's split partials and its (sequence, KV head) counters."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    if index not in _attn_scratch:
        with torch.cuda.device(index):
            _attn_scratch[index] = (torch.empty(_ATTN_SCRATCH_FLOATS, dtype=torch.float32, device="cuda"),
                                    torch.zeros(_ATTN_COUNTERS, dtype=torch.int32, device="cuda"))
    return _attn_scratch[index]


def attention_mma_block_queries() -> int:
    lib = build.load("attention_mma")
    lib.lb_attention_mma_block_queries.restype = c_int
    return lib.lb_attention_mma_block_queries()


def attention_prefill_bf16(q, k_pool, v_pool, out, block_table, cu_q, ctx_len, tile_seq, tile_q0, n_tiles, q_heads,
                           kv_heads, dim, page_tokens, scale, window=0):
    """Tensor-core paged attention for prompt portions: tiles of 64 queries, any number of queries per sequence."""
    for name, t in (("q", q), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _need(t, torch.int32, name)
    fn = _fn("attention_mma", "lb_attention_prefill_bf16",
             [c_void_p] * 5 + [c_int] + [c_void_p] * 4 + [c_int] * 5 + [c_float, c_int, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
              _ptr(ctx_len), _ptr(tile_seq), _ptr(tile_q0), n_tiles, q_heads, kv_heads, dim, page_tokens, float(scale),
              int(window), _stream()), "attention_prefill_bf16")
    return out


def decode_plan(n_seqs: int, q_heads: int, kv_heads: int, dim: int, max_context: int, sm_count: int,
                mean_context: int | None = None) -> tuple[int, int]:
    """(splits, stages): how many ways to split the context of a decode step, and which kernel variant.

    A block is one (sequence, KV head, split). With three K/V tiles in shared memory two blocks fit an
    SM; the variant with two tiles fits three (head size 128, at most 8 heads per KV head) but each
    block is slower (about 1.15x per tile). Blocks run in rounds of blocks-per-SM x SMs. With head size
    128 the kernel runs 2, 4 or 8 splits as a thread-block cluster that merges through distributed
    shared memory (16 where all the launch's blocks still fit one per SM: a single sequence, 8.7
    against 10.6 us at 3,072 keys; two sequences 16.5 against 12.1 us, so not there); more splits merge
    through scratch memory, which costs more. The plan is the one
    with the lowest estimate rounds x (64-key tiles per split + overhead in tiles): 4 for a cluster,
    10 for the scratch merge. That fits what was measured at 3,072 keys (sequences: best splits)
    1: 8, 4: 8, 8: 4, 16: 2, 24: 4, 32: 1, 40: 4, 48: 2, 128: 2, one sequence of 32,768 keys: 32 or
    more through scratch memory, and 64 sequences: 4 splits with three blocks an SM (148 us against
    158 us unsplit with two).

    `mean_context`: the sequences' mean length where it is known to be well below the longest (more
    than 1.5 times). The longest sequence's blocks then run on alone at a lone block's rate after the
    others have finished, so the context is cut further, into about 7 blocks an SM (at least 12 tiles
    each), with three blocks an SM as soon as two do not hold them all. Measured with lengths spread
    evenly over 0.1..1 of 8,192 keys (us, the plan for equal lengths against this one): 8 sequences
    54 -> 47, 16: 106 -> 80, 32: 219 -> 136; over 0.1..1 of 3,072 keys: 16: 41 -> 36, 32: 79 -> 56."""
    natural = n_seqs * kv_heads
    want = max(1, 2 * sm_count // natural)                    # all blocks resident at once, two per SM
    splits = min(want, 128, max(1, max_context // 192))       # at least three 64-key tiles per split
    while splits > 1 and n_seqs * q_heads * splits * (dim + 2) > _ATTN_SCRATCH_FLOATS:
        splits -= 1
    if dim != 128:
        return splits, 3
    tiles = max(1, -(-max_context // 64))

    def estimate(count: int, overhead: int, per_sm: int = 2, tile_cost: float = 1.0) -> float:
        return -(-natural * count // (per_sm * sm_count)) * (-(-tiles // count) * tile_cost + overhead)

    clustered = [c for c in (1, 2, 4, 8) if c <= tiles]
    if 16 <= tiles // 3 and natural * 16 <= sm_count:
        clustered.append(16)
    best = min(clustered, key=lambda c: (estimate(c, 4), c))
    plan, cost = (best, 3), estimate(best, 4)
    if splits > 8 and estimate(splits, 10) < cost:
        plan, cost = (splits, 3), estimate(splits, 10)
    skewed = mean_context is not None and 2 * max_context > 3 * max(1, mean_context)
    if skewed and q_heads // kv_heads <= 8 and 8 * natural > 2 * sm_count and 10 * natural < 34 * sm_count:
        count = 1
        while count < 8 and 2 * count * count * natural * natural <= (7 * sm_count) ** 2:   # nearest power of two to 7 SMs / natural
            count *= 2
        while count > 1 and tiles // count < 12:
            count //= 2
        if count >= 2:
            return (count, 3) if natural * count <= 2 * sm_count else (count, 2)
    if 10 * natural >= 17 * sm_count and natural <= 2 * sm_count and tiles >= 64 and q_heads // kv_heads <= 8:
        # just under two blocks an SM, long contexts: four splits with three blocks an SM measured
        # 200 against 225 us (32 sequences of 8,192 keys; at 3,072 keys the two are equal)
        return 4, 2
    if natural > 2 * sm_count and q_heads // kv_heads <= 8:
        # more blocks than two per SM hold at once: three slower blocks an SM may finish sooner
        packed = min((c for c in (1, 2, 4, 8) if c <= tiles), key=lambda c: (estimate(c, 4, 3, 1.15), c))
        if estimate(packed, 4, 3, 1.15) < cost:
            plan = (packed, 2)
    return plan


def decode_splits(n_seqs: int, q_heads: int, kv_heads: int, dim: int, max_context: int, sm_count: int) -> int:
    return decode_plan(n_seqs, q_heads, kv_heads, dim, max_context, sm_count)[0]


def attention_decode_bf16(q, k_pool, v_pool, out, block_table, cu_q, ctx_len, seq_list, n_seqs, q_heads, kv_heads, dim,
                          page_tokens, scale, window=0, splits=1, stages=3):
    """Tensor-core paged attention for sequences with one new token each, the context split `splits` ways
    (`stages` 2: the variant that fits three blocks an SM, see `decode_plan`)."""
    for name, t in (("q", q), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    if seq_list is not None:
        _need(seq_list, torch.int32, "seq_list")
    partials, counters = attention_scratch(q.device)
    fn = _fn("attention_mma", "lb_attention_decode_bf16",
             [c_void_p] * 5 + [c_int] + [c_void_p] * 3 + [c_int] * 5 + [c_float, c_int, c_int, c_void_p, c_long, c_void_p,
                                                                        c_int, c_int, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
              _ptr(ctx_len), _ptr(seq_list), n_seqs, q_heads, kv_heads, dim, page_tokens, float(scale), int(window),
              int(splits), _ptr(partials), partials.numel(), _ptr(counters), counters.numel(), int(stages), _stream()),
           "attention_decode_bf16")
    return out


# ---- attention on tcgen05 (head size 128, pages of 8..128 tokens dividing 128)
TCGEN05_TILE = 128
_pool_maps: dict[tuple, object] = {}


def attention_tcgen05_takes_heads(q_heads: int, kv_heads: int, dim: int) -> bool:
    """Whether the tcgen05 prompt attention has a kernel for these heads (whatever the page size)."""
    return dim == 128 and kv_heads > 0 and q_heads % kv_heads == 0 and q_heads // kv_heads <= 128


def attention_tcgen05_supports(q_heads: int, kv_heads: int, dim: int, page_tokens: int) -> bool:
    return (attention_tcgen05_takes_heads(q_heads, kv_heads, dim)
            and page_tokens >= 8 and page_tokens % 8 == 0 and 128 % page_tokens == 0)


def _pool_map(pool: torch.Tensor):
    """The TMA tensor map of a cache group's pool [layers, 2, pages, kv_heads, page_tokens, dim], made once."""
    key = (pool.data_ptr(), tuple(pool.shape))
    blob = _pool_maps.get(key)
    if blob is None:
        _need(pool, torch.bfloat16, "pool")
        layers, two, pages, kv_heads, page_tokens, dim = pool.shape
        blob = (ctypes.c_ubyte * 128)()
        fn = _fn("attention_tcgen05", "lb_attention_tcgen05_pool_map", [c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int])
        code = fn(ctypes.addressof(blob), _ptr(pool), layers * two, pages, kv_heads, page_tokens, dim)
        if code:
            raise ValueError(f"attention_tcgen05: cannot describe the pool to TMA ({_REFUSALS.get(code, code)})")
        _pool_maps[key] = blob
    return blob


def attention_tcgen05_status() -> int:
    """0, or which bounded wait of the tensor-core attention ran out. Synchronises; clears the code."""
    lib = build.load("attention_tcgen05")
    lib.lb_attention_tcgen05_status.restype = c_int
    torch.cuda.synchronize()
    return lib.lb_attention_tcgen05_status()


def attention_tcgen05_prefill(q, pool, layer, out, block_table, cu_q, ctx_len, tile_seq, tile_q0, n_tiles, q_heads,
                              kv_heads, dim, page_tokens, scale, window=0):
    """Prompt portions on tcgen05: tiles of 128 queries; pool is the cache group's whole pool."""
    for name, t in (("q", q), ("out", out)):
        _need(t, torch.bfloat16, name)
    for name, t in (("block_table", block_table), ("cu_q", cu_q), ("ctx_len", ctx_len), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _need(t, torch.int32, name)
    fn = _fn("attention_tcgen05", "lb_attention_tcgen05_prefill",
             [c_void_p, c_long, c_void_p, c_int, c_void_p, c_void_p, c_int] + [c_void_p] * 4 + [c_int] * 5 +
             [c_float, c_int, c_void_p])
    _check(fn(_ptr(q), q.shape[0], ctypes.addressof(_pool_map(pool)), int(layer), _ptr(out), _ptr(block_table),
              block_table.shape[1], _ptr(cu_q), _ptr(ctx_len), _ptr(tile_seq), _ptr(tile_q0), n_tiles, q_heads, kv_heads,
              dim, page_tokens, float(scale), int(window), _stream()), "attention_tcgen05_prefill")
    return out


def attention_bf16(q, cache, out, block_table, batch, q_heads, kv_heads, dim, page_tokens, scale, window):
    """The bfloat16 path's attention for one step: prompt portions go through the tcgen05 tile kernel
    where it takes the sizes (head size 128, pages of 8..128 tokens), else through the mma.sync
    one; single tokens, alone or beside prompt portions, go through the split decode kernel."""
    if batch.all_decode and q_heads // kv_heads <= 16:
        sms = gemm_scratch(q.device)[2]
        # planned for the step's own lengths; a captured step for its class of steps (the widest context
        # its block table can describe, with the mean that the class stands for)
        widest = min(batch.plan_max_ctx or block_table.shape[1] * page_tokens, block_table.shape[1] * page_tokens)
        splits, stages = decode_plan(batch.n_seqs, q_heads, kv_heads, dim, widest, sms, batch.plan_mean_ctx or None)
        attention_decode_bf16(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, None,
                              batch.n_seqs, q_heads, kv_heads, dim, page_tokens, scale, window, splits, stages)
        return
    tiles_of = batch.tiles
    if batch.n_decode_seqs > 0 and q_heads // kv_heads <= 16:
        # a mixed step: the sequences with a single token go through the decode kernel (a tile kernel
        # would spend a whole tile of queries on each), the prompt portions through the tile kernel
        sms = gemm_scratch(q.device)[2]
        splits, stages = decode_plan(batch.n_decode_seqs, q_heads, kv_heads, dim, batch.decode_max_ctx, sms,
                                     batch.plan_mean_ctx or None)
        attention_decode_bf16(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, batch.decode_seqs,
                              batch.n_decode_seqs, q_heads, kv_heads, dim, page_tokens, scale, window, splits, stages)
        tiles_of = batch.portion_tiles
    if cache.pool is not None and attention_tcgen05_supports(q_heads, kv_heads, dim, page_tokens):
        tiles = tiles_of[TCGEN05_TILE]
        attention_tcgen05_prefill(q, cache.pool, cache.layer, out, block_table, batch.cu_q, batch.ctx_len, tiles.tile_seq,
                                  tiles.tile_q0, tiles.count, q_heads, kv_heads, dim, page_tokens, scale, window)
        return
    tiles = tiles_of[attention_mma_block_queries()]
    attention_prefill_bf16(q, cache.k_pool, cache.v_pool, out, block_table, batch.cu_q, batch.ctx_len, tiles.tile_seq,
                           tiles.tile_q0, tiles.count, q_heads, kv_heads, dim, page_tokens, scale, window)
