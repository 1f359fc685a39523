// Paged grouped-query attention for bfloat16 on tensor cores (mma.sync m16n8k16, 32-bit
// accumulation, 32-bit softmax), read straight from the block table. The reference gathers the
// history out of its pool and calls a library kernel for prompts (layover/model.py:84-90) and runs
// one program per (sequence, query head) without splitting for decode
// (layover/kernels/triton_decode.py:39-119, which re-reads each KV head once per query head).
//
// Two kernels share the tile code:
//   prefill  one block per (tile of 64 queries of one sequence, query head); its four warps own 16
//            query rows each and walk the keys in tiles of 64 with a two-stage cp.async pipeline;
//            the causal mask (and a window) is applied from absolute positions.
//   decode   one block per (sequence with a single new token, KV head, split of the context); the
//            query heads that share the KV head are the rows of one 16-row MMA tile, so every key
//            and value is read once for the whole group; the four warps take 16 keys each of every
//            64-key tile and are merged at the end. With more than one split each block writes
//            (max, sum, unnormalised output) to scratch memory and the block that arrives last at
//            the (sequence, KV head) counter merges the splits in order and resets the counter.
//
// Keys outside [first visible key, context length) are loaded as zeros and masked by replacing
// their scores, so stale or non-finite page contents cannot reach a result. Head sizes are
// multiples of 16 up to 256 (a runtime value under a compile-time bound of 128 or 256).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int BKEYS = 64;     // keys per tile
constexpr int BQ = 64;        // queries per prefill block (16 per warp)
constexpr int PAD = 8;        // bf16 of padding per shared-memory row: rows 16 bytes apart modulo 128

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte async copy; bytes == 0 writes zeros instead of reading
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

constexpr int TABLE_CACHE = 1024;   // block-table entries a prompt block keeps in shared memory
constexpr int DECODE_TABLE_CACHE = 256;   // ... and a decode block (4,096 keys at pages of 16; the rest is read from global memory)

// The pages of keys [first_key, last_key] copied to shared memory once, so that the tile loads do
// not wait on a dependent global read each; entries past the cache are read from global memory.
struct TableSlice {
  const int* table;
  const int* cached;
  int first_page, capacity;
  __device__ __forceinline__ int page(int index) const {
    const int local = index - first_page;
    return (local >= 0 && local < capacity) ? cached[local] : table[index];
  }
};

__device__ __forceinline__ TableSlice cache_table(int* cached, int capacity, const int* __restrict__ table, int first_key,
                                                   int last_key, int page_tokens) {
  const int first_page = first_key / page_tokens, n = min(capacity, last_key / page_tokens - first_page + 1);
  for (int i = threadIdx.x; i < n; i += THREADS) cached[i] = table[first_page + i];
  return TableSlice{table, cached, first_page, capacity};
}

// Copies keys [tile * 64, +64) of one KV head into shared memory rows of (dim + PAD) bf16; keys
// outside [key_lo, key_hi) become zeros. Consecutive threads take consecutive 16-byte pieces, and
// a page of one head is one contiguous run, so every request is a full line.
struct TileShape {
  int kv_heads, kv_head, dim, page_tokens;
  int chunk_shift;   // log2(dim / 8) when that is a power of two, else -1
  int page_shift;    // log2(page_tokens) when that is a power of two, else -1
};

__device__ __forceinline__ void load_kv_tile(bf16* k_s, bf16* v_s, const bf16* __restrict__ k_pool,
                                             const bf16* __restrict__ v_pool, const TableSlice& pages,
                                             int tile, int key_lo, int key_hi, const TileShape& shape) {
  const int dim = shape.dim, stride = dim + PAD, page_tokens = shape.page_tokens;
  if (shape.chunk_shift >= 0 && shape.page_shift >= 0) {
    // shifts and masks only: the thread's piece of a row and its first key are fixed for the kernel
    const int c8 = (threadIdx.x & ((1 << shape.chunk_shift) - 1)) * 8;
    const int keys_per_pass = THREADS >> shape.chunk_shift;
#pragma unroll 4
    for (int j = threadIdx.x >> shape.chunk_shift; j < BKEYS; j += keys_per_pass) {
      const int key = tile * BKEYS + j;
      const bool live = key >= key_lo && key < key_hi;
      size_t at = 0;
      if (live) {
        const int index = key >> shape.page_shift;
        at = (((size_t)pages.page(index) * shape.kv_heads + shape.kv_head) * page_tokens + (key & (page_tokens - 1))) * dim + c8;
      }
      cp_async16(k_s + j * stride + c8, k_pool + at, live ? 16 : 0);
      cp_async16(v_s + j * stride + c8, v_pool + at, live ? 16 : 0);
    }
    return;
  }
  const int chunks = dim >> 3;
  for (int i = threadIdx.x; i < BKEYS * chunks; i += THREADS) {
    const int j = i / chunks, c = i - j * chunks;
    const int key = tile * BKEYS + j;
    const bool live = key >= key_lo && key < key_hi;
    size_t at = 0;
    if (live) {
      const int index = key / page_tokens;
      at = (((size_t)pages.page(index) * shape.kv_heads + shape.kv_head) * page_tokens + (key - index * page_tokens)) * dim + c * 8;
    }
    cp_async16(k_s + j * stride + c * 8, k_pool + at, live ? 16 : 0);
    cp_async16(v_s + j * stride + c * 8, v_pool + at, live ? 16 : 0);
  }
}

// ------------------------------------------------------------------------------- one warp, one tile
__device__ __forceinline__ void ldmatrix_x4_at(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans_at(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// The 16 query rows of one warp against PAIRS * 16 keys of a tile in shared memory:
// scores, mask, running maximum and sum, P V. `k_addr` / `v_addr` are shared-memory byte addresses
// of the warp's first key row plus this lane's ldmatrix offset; with EXACT the head size equals
// MAX_DIM and every address offset is a constant. UPPER false skips the softmax of rows 8..15
// (decode with at most 8 query heads per KV head). `masked` false skips the comparisons for a
// tile that every row sees completely. Scores stay unscaled; the scale enters the exponent.
template <int MAX_DIM, bool EXACT, int PAIRS, bool UPPER>
__device__ __forceinline__ void warp_tile(const uint32_t (&qf)[MAX_DIM / 16][4], uint32_t k_addr, uint32_t v_addr,
                                          int dim, float (&o)[MAX_DIM / 8][4], float (&m_run)[2], float (&l_run)[2],
                                          bool masked, int key0, int p0, int p1, int key_lo, int window, float c,
                                          int t) {
  constexpr int KSTEPS = MAX_DIM / 16, NT_O = MAX_DIM / 8, NT_S = PAIRS * 2;
  const int dk = EXACT ? KSTEPS : (dim >> 4);
  const uint32_t row_bytes = (uint32_t)((EXACT ? MAX_DIM : dim) + PAD) * 2;
  float s[NT_S][4];
#pragma unroll
  for (int n = 0; n < NT_S; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
  // loads in batches of four before the MMAs that use them, so that neither waits on the other
  if (PAIRS >= 4) {
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
      if (EXACT || k < dk) {
#pragma unroll
        for (int n0 = 0; n0 < PAIRS; n0 += 4) {
          uint32_t b[4][4];
#pragma unroll
          for (int u = 0; u < 4; ++u) ldmatrix_x4_at(b[u], k_addr + (n0 + u) * 16 * row_bytes + k * 32);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            mma_bf16(s[2 * (n0 + u)], qf[k], b[u][0], b[u][1]);
            mma_bf16(s[2 * (n0 + u) + 1], qf[k], b[u][2], b[u][3]);
          }
        }
      }
    }
  } else {
#pragma unroll
    for (int k0 = 0; k0 < KSTEPS; k0 += 4) {
#pragma unroll
      for (int n2 = 0; n2 < PAIRS; ++n2) {
        uint32_t b[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (EXACT || k0 + u < dk) ldmatrix_x4_at(b[u], k_addr + n2 * 16 * row_bytes + (k0 + u) * 32);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (EXACT || k0 + u < dk) {
            mma_bf16(s[2 * n2], qf[k0 + u], b[u][0], b[u][1]);
            mma_bf16(s[2 * n2 + 1], qf[k0 + u], b[u][2], b[u][3]);
          }
        }
      }
    }
  }
  if (masked) {
#pragma unroll
    for (int n = 0; n < NT_S; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (!UPPER && e >= 2) continue;
        const int key = key0 + n * 8 + 2 * t + (e & 1);
        const int p = e < 2 ? p0 : p1;
        const bool seen = key <= p && key >= key_lo && (window <= 0 || p - key < window);
        if (!seen) s[n][e] = -INFINITY;
      }
    }
  }
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int n = 0; n < NT_S; ++n) {
    tile_max[0] = fmaxf(tile_max[0], fmaxf(s[n][0], s[n][1]));
    if (UPPER) tile_max[1] = fmaxf(tile_max[1], fmaxf(s[n][2], s[n][3]));
  }
  float alpha[2] = {1.f, 1.f}, neg_base[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < (UPPER ? 2 : 1); ++r) {
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
    const float m_new = fmaxf(m_run[r], tile_max[r]);
    const float base = m_new == -INFINITY ? 0.f : m_new;
    alpha[r] = fast_exp2((m_run[r] - base) * c);      // exp2(-inf) = 0 on the first tile
    neg_base[r] = -base * c;
    m_run[r] = m_new;
  }
  float tile_sum[2] = {0.f, 0.f};
  uint32_t pf[PAIRS][4];
#pragma unroll
  for (int n = 0; n < NT_S; ++n) {
    const float e0 = fast_exp2(fmaf(s[n][0], c, neg_base[0])), e1 = fast_exp2(fmaf(s[n][1], c, neg_base[0]));
    tile_sum[0] += e0 + e1;
    pf[n >> 1][(n & 1) * 2] = pack_bf16(e0, e1);
    if (UPPER) {
      const float e2 = fast_exp2(fmaf(s[n][2], c, neg_base[1])), e3 = fast_exp2(fmaf(s[n][3], c, neg_base[1]));
      tile_sum[1] += e2 + e3;
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(e2, e3);
    } else {
      pf[n >> 1][(n & 1) * 2 + 1] = 0u;
    }
  }
  l_run[0] = l_run[0] * alpha[0] + tile_sum[0];
  if (UPPER) l_run[1] = l_run[1] * alpha[1] + tile_sum[1];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) {
    if (EXACT || n * 8 < dim) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
      if (UPPER) { o[n][2] *= alpha[1]; o[n][3] *= alpha[1]; }
    }
  }
#pragma unroll
  for (int kk = 0; kk < PAIRS; ++kk) {
#pragma unroll
    for (int n0 = 0; n0 < NT_O / 2; n0 += 4) {
      uint32_t b[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (EXACT || n0 + u < dk) ldmatrix_x4_trans_at(b[u], v_addr + kk * 16 * row_bytes + (n0 + u) * 32);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (EXACT || n0 + u < dk) {
          mma_bf16(o[2 * (n0 + u)], pf[kk], b[u][0], b[u][1]);
          mma_bf16(o[2 * (n0 + u) + 1], pf[kk], b[u][2], b[u][3]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------- prefill
template <int MAX_DIM, bool EXACT>
__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                         bf16* __restrict__ out, const int* __restrict__ block_table, int table_width,
                         const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                         const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, int q_heads, int kv_heads,
                         int dim_arg, int page_tokens, float scale_log2, int window, int chunk_shift, int page_shift) {
  constexpr int KSTEPS = MAX_DIM / 16, NT_O = MAX_DIM / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int dim = EXACT ? MAX_DIM : dim_arg;
  const int stride = dim + PAD;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);
  bf16* k_s = q_s + BQ * stride;            // [2][BKEYS][stride]
  bf16* v_s = k_s + 2 * BKEYS * stride;
  __shared__ int table_cache[TABLE_CACHE];
  pdl_launch_dependents();
  pdl_wait();

  const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x], head = blockIdx.y;
  const int kv_head = head / (q_heads / kv_heads);
  const int row0 = cu_q[seq], q_len = cu_q[seq + 1] - row0, ctx = ctx_len[seq];
  const int start = ctx - q_len;
  const int n_q = min(BQ, q_len - q0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int* table = block_table + (size_t)seq * table_width;
  const int dk = dim >> 4;

  const int p_first = start + q0, p_last = p_first + n_q - 1;
  const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int tile_lo = key_lo / BKEYS, tile_hi = p_last / BKEYS;
  const TableSlice pages = cache_table(table_cache, TABLE_CACHE, table, key_lo, p_last, page_tokens);
  const TileShape shape{kv_heads, kv_head, dim, page_tokens, chunk_shift, page_shift};
  __syncthreads();

  {  // the block's queries
    const int chunks = dim >> 3;
    for (int i = threadIdx.x; i < BQ * chunks; i += THREADS) {
      const int r = i / chunks, c = i % chunks;
      const bool live = r < n_q;
      const bf16* src = q + ((size_t)(row0 + q0 + (live ? r : 0)) * q_heads + head) * dim + c * 8;
      cp_async16(q_s + r * stride + c * 8, src, live ? 16 : 0);
    }
  }
  load_kv_tile(k_s, v_s, k_pool, v_pool, pages, tile_lo, key_lo, p_last + 1, shape);
  cp_async_commit();

  uint32_t qf[KSTEPS][4];
  float o[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int p_warp = p_first + warp * 16;                   // position of the warp's first row
  const int p0 = p_warp + g, p1 = p_warp + g + 8;           // rows past n_q compute harmlessly
  // lane offsets of the ldmatrix rows (bytes): K rows by key, V rows by key with the d-chunk swapped in
  const uint32_t k_lane = (uint32_t)(((lane >> 4) * 8 + (lane & 7)) * stride + ((lane >> 3) & 1) * 8) * 2;
  const uint32_t v_lane = (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * stride + (lane >> 4) * 8) * 2;
  const uint32_t k_base = smem_u32(k_s) + k_lane, v_base = smem_u32(v_s) + v_lane;
  const uint32_t buf_bytes = (uint32_t)BKEYS * stride * 2;

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int buf = (tile - tile_lo) & 1;
    if (tile < tile_hi) {
      load_kv_tile(k_s + (buf ^ 1) * BKEYS * stride, v_s + (buf ^ 1) * BKEYS * stride, k_pool, v_pool, pages, tile + 1,
                   key_lo, p_last + 1, shape);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (tile == tile_lo) {
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k)
        if (EXACT || k < dk) ldmatrix_x4(qf[k], q_s + (warp * 16 + (lane & 15)) * stride + k * 16 + (lane >> 4) * 8);
    }
    // a warp whose rows all lie before this tile has nothing to do in it
    if (tile * BKEYS <= p_warp + 15) {
      // every row of the warp sees the whole tile unless it reaches past the first row's position,
      // starts before the first visible key or a window cuts it
      const bool masked = tile * BKEYS + BKEYS - 1 > p_warp || tile * BKEYS < key_lo || window > 0;
      warp_tile<MAX_DIM, EXACT, BKEYS / 16, true>(qf, k_base + buf * buf_bytes, v_base + buf * buf_bytes, dim, o, m_run,
                                                  l_run, masked, tile * BKEYS, p0, p1, key_lo, window, scale_log2, t);
    }
    __syncthreads();   // the buffer may be overwritten by the next iteration's prefetch
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + 8 * r;
    if (row >= n_q) continue;
    const float inv = 1.0f / l_run[r];
    bf16* dst = out + ((size_t)(row0 + q0 + row) * q_heads + head) * dim;
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      if (EXACT || n * 8 < dim)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_bf16(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------------------- decode
// Rows 0..group-1 of the 16-row tile are the query heads of one KV head (group <= 16).
// CLUSTER: the `splits` blocks of a (sequence, KV head) are one thread-block cluster (grid z =
// cluster z = splits). Instead of writing partial results to scratch memory and leaving the merge
// to the block that arrives last at a counter, every block owns a share of the group's outputs:
// after a first cluster barrier (every block has left its loop, so the tile buffers are free) each
// block sends its partial values of a share to the share's owner and its maxima and sums to
// everyone, through distributed shared memory; after a second barrier the owners add their shares
// in split order and store them.
// STAGES: K/V tiles of a block in shared memory. Three keep a block's own stream going (two loads in
// flight); with two a block is slower but three blocks share an SM instead of two, which wins once a
// launch has more blocks than two per SM can hold at once (12 warps an SM hide the MMAs' latency
// better than 8; measured at 64 sequences of 3,072 keys: 148 us against 158 us).
template <int MAX_DIM, bool EXACT, bool UPPER, bool CLUSTER = false, int STAGES = 3>
__global__ void __launch_bounds__(THREADS, STAGES == 2 ? 3 : 2)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        bf16* __restrict__ out, const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                        const int* __restrict__ seq_list, int q_heads, int kv_heads, int dim_arg, int page_tokens,
                        float scale_log2, int window, int splits, float* __restrict__ partials,
                        unsigned* __restrict__ counters, int chunk_shift, int page_shift) {
  constexpr int KSTEPS = MAX_DIM / 16, NT_O = MAX_DIM / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int dim = EXACT ? MAX_DIM : dim_arg;
  const int stride = dim + PAD;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);          // [16][stride]
  bf16* k_s = q_s + 16 * stride;                          // [STAGES][BKEYS][stride]
  bf16* v_s = k_s + STAGES * BKEYS * stride;
  __shared__ unsigned last_flag;
  __shared__ int table_cache[DECODE_TABLE_CACHE];
  // Lengths and block tables are written when the step begins, and the keys of earlier positions by
  // earlier steps: the block reads them, and requests its first tiles, while the kernel before it
  // still runs. What that kernel writes, the query and the tile that holds the newest key, is
  // fetched after the wait.
  pdl_launch_dependents();

  const int seq = seq_list ? seq_list[blockIdx.x] : blockIdx.x;
  const int kv_head = blockIdx.y, split = blockIdx.z;
  const int group = q_heads / kv_heads, head0 = kv_head * group;
  const int row = cu_q[seq];                               // the sequence's single query row
  const int ctx = ctx_len[seq], p = ctx - 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int* table = block_table + (size_t)seq * table_width;
  const int dk = dim >> 4;

  const int key_lo = window > 0 ? max(0, p - window + 1) : 0;
  const int first_tile = key_lo / BKEYS, n_tiles = p / BKEYS + 1 - first_tile;
  const int per_split = (n_tiles + splits - 1) / splits;
  const int tile_begin = first_tile + split * per_split;
  const int tile_end = min(first_tile + n_tiles, tile_begin + per_split);
  const TableSlice pages = cache_table(table_cache, DECODE_TABLE_CACHE, table, max(key_lo, tile_begin * BKEYS),
                                       min(p, max(tile_end, tile_begin + 1) * BKEYS - 1), page_tokens);
  const TileShape shape{kv_heads, kv_head, dim, page_tokens, chunk_shift, page_shift};
  __syncthreads();

  const int newest_tile = p / BKEYS;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (tile_begin + s < tile_end && tile_begin + s != newest_tile)
      load_kv_tile(k_s + s * BKEYS * stride, v_s + s * BKEYS * stride, k_pool, v_pool, pages, tile_begin + s, key_lo, ctx,
                   shape);
    cp_async_commit();
  }
  pdl_wait();
  {
    const int chunks = dim >> 3;
    for (int i = threadIdx.x; i < 16 * chunks; i += THREADS) {
      const int r = i / chunks, c = i % chunks;
      const bool live = r < group;
      const bf16* src = q + ((size_t)row * q_heads + head0 + (live ? r : 0)) * dim + c * 8;
      cp_async16(q_s + r * stride + c * 8, src, live ? 16 : 0);
    }
  }
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (tile_begin + s < tile_end && tile_begin + s == newest_tile)
      load_kv_tile(k_s + s * BKEYS * stride, v_s + s * BKEYS * stride, k_pool, v_pool, pages, tile_begin + s, key_lo, ctx,
                   shape);
  }
  cp_async_commit();     // the query and the held tile: one more group than the ring has stages

  uint32_t qf[KSTEPS][4];
  float o[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const uint32_t k_lane = (uint32_t)((warp * 16 + (lane >> 4) * 8 + (lane & 7)) * stride + ((lane >> 3) & 1) * 8) * 2;
  const uint32_t v_lane = (uint32_t)((warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * stride + (lane >> 4) * 8) * 2;
  const uint32_t k_base = smem_u32(k_s) + k_lane, v_base = smem_u32(v_s) + v_lane;
  const uint32_t buf_bytes = (uint32_t)BKEYS * stride * 2;

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int i = tile - tile_begin, buf = i % STAGES;
    if (tile + STAGES - 1 < tile_end) {
      const int nb = (i + STAGES - 1) % STAGES;
      load_kv_tile(k_s + nb * BKEYS * stride, v_s + nb * BKEYS * stride, k_pool, v_pool, pages, tile + STAGES - 1, key_lo,
                   ctx, shape);
    }
    cp_async_commit();
    // the first tile also waits for the group of the query, which was committed after the ring's
    if (i == 0) cp_async_wait<1>(); else cp_async_wait<STAGES - 1>();
    __syncthreads();
    if (i == 0) {
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k)
        if (EXACT || k < dk) ldmatrix_x4(qf[k], q_s + (lane & 15) * stride + k * 16 + (lane >> 4) * 8);
    }
    // only the tile that holds the last key, or the first visible one, needs the comparisons
    const bool masked = tile * BKEYS + BKEYS - 1 > p || tile * BKEYS < key_lo;
    warp_tile<MAX_DIM, EXACT, 1, UPPER>(qf, k_base + buf * buf_bytes, v_base + buf * buf_bytes, dim, o, m_run, l_run, masked,
                                        tile * BKEYS + warp * 16, p, p, key_lo, 0, scale_log2, t);
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }

  // ---- merge the four warps through shared memory (the tile buffers are free now)
  __syncthreads();
  float* merge = reinterpret_cast<float*>(smem_raw);      // [WARPS][16][dim + 2]: output, then max, then sum
  const int mstride = dim + 2;
#pragma unroll
  for (int r = 0; r < (UPPER ? 2 : 1); ++r) {
    float* dst = merge + ((size_t)warp * 16 + g + 8 * r) * mstride;
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      if (EXACT || n * 8 < dim) { dst[n * 8 + 2 * t] = o[n][2 * r]; dst[n * 8 + 2 * t + 1] = o[n][2 * r + 1]; }
    }
    if (t == 0) { dst[dim] = m_run[r]; dst[dim + 1] = l_run[r]; }
  }
  __syncthreads();
  const float c = scale_log2;
  if (CLUSTER) {
    const int total = group * dim, per = (total + splits - 1) / splits;
    float* recv_acc = merge + (size_t)WARPS * 16 * mstride;            // [splits][per]: this block's share, from every split
    float* recv_ml = recv_acc + (size_t)splits * per;                   // [splits][group][2]
    lb_cluster_barrier();
    for (int i = threadIdx.x; i < total; i += THREADS) {
      const int r = i / dim, col = i % dim;
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m_all = fmaxf(m_all, merge[((size_t)w * 16 + r) * mstride + dim]);
      const float base = m_all == -INFINITY ? 0.f : m_all;
      float acc = 0.f, l_all = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float* src = merge + ((size_t)w * 16 + r) * mstride;
        const float f = fast_exp2((src[dim] - base) * c);
        acc += src[col] * f;
        l_all += src[dim + 1] * f;
      }
      const int owner = i / per;
      lb_store_remote(lb_map_to_rank(smem_u32(recv_acc + (size_t)split * per + (i - owner * per)), owner), acc);
      if (col == 0) {
        for (int peer = 0; peer < splits; ++peer) {
          const uint32_t dst = lb_map_to_rank(smem_u32(recv_ml + ((size_t)split * group + r) * 2), peer);
          lb_store_remote(dst, m_all);
          lb_store_remote(dst + 4, l_all);
        }
      }
    }
    lb_cluster_barrier();
    for (int k = threadIdx.x; k < per; k += THREADS) {
      const int i = split * per + k;
      if (i >= total) break;
      const int r = i / dim, col = i % dim;
      float m_max = -INFINITY;
      for (int s2 = 0; s2 < splits; ++s2) m_max = fmaxf(m_max, recv_ml[((size_t)s2 * group + r) * 2]);
      const float base = m_max == -INFINITY ? 0.f : m_max;
      float acc = 0.f, l_all = 0.f;
      for (int s2 = 0; s2 < splits; ++s2) {
        const float f = fast_exp2((recv_ml[((size_t)s2 * group + r) * 2] - base) * c);
        acc += recv_acc[(size_t)s2 * per + k] * f;
        l_all += recv_ml[((size_t)s2 * group + r) * 2 + 1] * f;
      }
      out[((size_t)row * q_heads + head0 + r) * dim + col] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
    }
    return;
  }
  const unsigned tile_id = blockIdx.x * gridDim.y + blockIdx.y;
  float* my_partial = partials ? partials + ((size_t)tile_id * splits + split) * group * mstride : nullptr;
  for (int i = threadIdx.x; i < group * dim; i += THREADS) {
    const int r = i / dim, col = i % dim;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m_all = fmaxf(m_all, merge[((size_t)w * 16 + r) * mstride + dim]);
    const float base = m_all == -INFINITY ? 0.f : m_all;
    float acc = 0.f, l_all = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float* src = merge + ((size_t)w * 16 + r) * mstride;
      const float f = fast_exp2((src[dim] - base) * c);
      acc += src[col] * f;
      l_all += src[dim + 1] * f;
    }
    if (splits == 1) {
      out[((size_t)row * q_heads + head0 + r) * dim + col] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
    } else {
      my_partial[r * mstride + col] = acc;
      if (col == 0) { my_partial[r * mstride + dim] = m_all; my_partial[r * mstride + dim + 1] = l_all; }
    }
  }
  if (splits == 1) return;

  // ---- the block that arrives last merges the splits in order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_flag = atomicAdd(&counters[tile_id], 1u) == (unsigned)splits - 1 ? 1u : 0u;
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  const float* all = partials + (size_t)tile_id * splits * group * mstride;
  // per (split, row): the factor that brings the split's sums to the common maximum, in shared
  // memory first, so that the loads of the second pass do not wait on one another
  float* factor = merge;                                   // [splits][group], then [group] sums
  float* l_total = merge + (size_t)splits * group;
  float* m_part = l_total + group;                         // [splits][group] maxima, then sums
  float* l_part = m_part + (size_t)splits * group;
  __syncthreads();
  for (int i = threadIdx.x; i < splits * group; i += THREADS) {   // every (split, row) is its own load
    const float* src = all + (size_t)i * mstride;
    m_part[i] = src[dim];
    l_part[i] = src[dim + 1];
  }
  __syncthreads();
  for (int r = threadIdx.x; r < group; r += THREADS) {
    float m_all = -INFINITY;
    for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, m_part[s * group + r]);
    const float base = m_all == -INFINITY ? 0.f : m_all;
    float l_all = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float f = fast_exp2((m_part[s * group + r] - base) * c);
      factor[s * group + r] = f;
      l_all += l_part[s * group + r] * f;
    }
    l_total[r] = l_all;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < group * dim; i += THREADS) {
    const int r = i / dim, col = i % dim;
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) acc += all[((size_t)s * group + r) * mstride + col] * factor[s * group + r];
    out[((size_t)row * q_heads + head0 + r) * dim + col] = __float2bfloat16_rn(l_total[r] > 0.f ? acc / l_total[r] : 0.f);
  }
  if (threadIdx.x == 0) counters[tile_id] = 0;
}

int exact_log2(int v) {
  int shift = 0;
  while ((1 << shift) < v) ++shift;
  return (1 << shift) == v ? shift : -1;
}
size_t prefill_smem(int dim) { return (size_t)(BQ + 4 * BKEYS) * (dim + PAD) * sizeof(bf16); }
size_t decode_smem(int dim, int stages = 3) {
  const size_t tiles = (size_t)(16 + 2 * stages * BKEYS) * (dim + PAD) * sizeof(bf16);
  const size_t merge = (size_t)WARPS * 16 * (dim + 2) * sizeof(float);
  return tiles > merge ? tiles : merge;
}
}  // namespace

LB_EXPORT int lb_attention_mma_block_queries() { return BQ; }

namespace {
template <typename Kernel> void allow_smem(Kernel kernel, size_t bytes) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}
void configure_once() {      // once per device: the attribute belongs to the device that is current
  static LbPerDeviceOnce once;
  if (!once.first()) return;
  allow_smem(attention_prefill_kernel<128, true>, prefill_smem(128));
  allow_smem(attention_prefill_kernel<128, false>, prefill_smem(128));
  allow_smem(attention_prefill_kernel<256, true>, prefill_smem(256));
  allow_smem(attention_prefill_kernel<256, false>, prefill_smem(256));
  allow_smem(attention_decode_kernel<128, true, false>, decode_smem(128));
  allow_smem(attention_decode_kernel<128, true, true>, decode_smem(128));
  allow_smem(attention_decode_kernel<128, false, true>, decode_smem(128));
  allow_smem(attention_decode_kernel<256, true, true>, decode_smem(256));
  allow_smem(attention_decode_kernel<256, false, true>, decode_smem(256));
  allow_smem(attention_decode_kernel<128, true, false, true>, decode_smem(128));
  allow_smem(attention_decode_kernel<128, true, true, true>, decode_smem(128));
  // clusters of 16 blocks (one sequence's context cut 16 ways) are beyond the portable size of 8
  cudaFuncSetAttribute(attention_decode_kernel<128, true, false, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  cudaFuncSetAttribute(attention_decode_kernel<128, true, true, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  cudaGetLastError();
  allow_smem(attention_decode_kernel<128, true, false, false, 2>, decode_smem(128, 2));
  allow_smem(attention_decode_kernel<128, true, false, true, 2>, decode_smem(128, 2));
}

// launches the decode kernel instantiation for this head size and group
template <typename... Args>
int launch_decode(int dim, int group, dim3 grid, size_t smem, cudaStream_t stream, Args... args) {
  if (dim == 128) {
    if (group <= 8) return lb_launch(attention_decode_kernel<128, true, false>, grid, dim3(THREADS), smem, stream, args...);
    return lb_launch(attention_decode_kernel<128, true, true>, grid, dim3(THREADS), smem, stream, args...);
  }
  if (dim < 128) return lb_launch(attention_decode_kernel<128, false, true>, grid, dim3(THREADS), smem, stream, args...);
  if (dim == 256) return lb_launch(attention_decode_kernel<256, true, true>, grid, dim3(THREADS), smem, stream, args...);
  return lb_launch(attention_decode_kernel<256, false, true>, grid, dim3(THREADS), smem, stream, args...);
}

// Whether the splits of this launch can run as clusters: head size 128, 2, 4 or 8 splits, and room
// for the received shares behind the warps' merge area.
bool decode_cluster_fits(int dim, int group, int splits, size_t smem) {
  if (dim != 128 || splits < 2 || splits > 16 || (splits & (splits - 1)) || !lb_cluster_reduce_enabled()) return false;
  const size_t per = ((size_t)group * dim + splits - 1) / splits;
  const size_t need = ((size_t)WARPS * 16 * (dim + 2) + splits * per + (size_t)splits * group * 2) * sizeof(float);
  return need <= smem;
}
template <typename... Args>
int launch_decode_cluster(int group, dim3 grid, size_t smem, cudaStream_t stream, Args... args) {
  if (group <= 8)
    return lb_launch_cluster(attention_decode_kernel<128, true, false, true>, grid, dim3(THREADS), smem, stream, grid.z, args...);
  return lb_launch_cluster(attention_decode_kernel<128, true, true, true>, grid, dim3(THREADS), smem, stream, grid.z, args...);
}
}  // namespace

// Prompt portions (any number of queries per sequence), listed as tiles of 64 queries.
LB_EXPORT int lb_attention_prefill_bf16(const void* q, const void* k_pool, const void* v_pool, void* out,
                                        const int* block_table, int table_width, const int* cu_q, const int* ctx_len,
                                        const int* tile_seq, const int* tile_q0, int n_tiles, int q_heads, int kv_heads,
                                        int dim, int page_tokens, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (dim <= 0 || dim % 16 || dim > 256 || kv_heads <= 0 || q_heads % kv_heads || q_heads > 65535) return LB_ERR_SIZE;
  configure_once();
  const size_t smem = prefill_smem(dim);
  const float scale_log2 = scale * 1.4426950408889634f;
  const int chunk_shift = (dim >> 3) <= THREADS ? exact_log2(dim >> 3) : -1, page_shift = exact_log2(page_tokens);
  dim3 grid(n_tiles, q_heads), block(THREADS);
  int code;
#define LB_PREFILL_ARGS (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, block_table, table_width, cu_q, \
                        ctx_len, tile_seq, tile_q0, q_heads, kv_heads, dim, page_tokens, scale_log2, window, chunk_shift, page_shift
  if (dim == 128) code = lb_launch(attention_prefill_kernel<128, true>, grid, block, smem, stream, LB_PREFILL_ARGS);
  else if (dim < 128) code = lb_launch(attention_prefill_kernel<128, false>, grid, block, smem, stream, LB_PREFILL_ARGS);
  else if (dim == 256) code = lb_launch(attention_prefill_kernel<256, true>, grid, block, smem, stream, LB_PREFILL_ARGS);
  else code = lb_launch(attention_prefill_kernel<256, false>, grid, block, smem, stream, LB_PREFILL_ARGS);
#undef LB_PREFILL_ARGS
  return code ? code : lb_last_error();
}

// Floats of scratch that `splits` splits of `n_seqs` sequences need.
LB_EXPORT long lb_attention_decode_scratch(int n_seqs, int q_heads, int dim, int splits) {
  return splits <= 1 ? 0 : (long)n_seqs * q_heads * splits * (dim + 2);
}

// Sequences with one new token each. `seq_list` (n_seqs indices into cu_q / ctx_len / block_table)
// may be null for "all of them in order". `stages` 2 asks for the variant with two K/V tiles a block in
// shared memory and three blocks an SM (for launches of more blocks than two per SM hold at once); it
// is honoured for head size 128 with at most 8 query heads per KV head, else three stages run. A sequence whose ctx_len is 0 (no key at all) gets zeros. `counters` (n_seqs * kv_heads, zero between launches) and
// `partials` are needed when splits > 1.
LB_EXPORT int lb_attention_decode_bf16(const void* q, const void* k_pool, const void* v_pool, void* out,
                                       const int* block_table, int table_width, const int* cu_q, const int* ctx_len,
                                       const int* seq_list, int n_seqs, int q_heads, int kv_heads, int dim,
                                       int page_tokens, float scale, int window, int splits, float* partials,
                                       long partial_floats, unsigned* counters, int n_counters, int stages,
                                       cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (dim <= 0 || dim % 16 || dim > 256 || kv_heads <= 0 || q_heads % kv_heads || q_heads / kv_heads > 16 ||
      kv_heads > 65535 || splits < 1 || splits > 65535)
    return LB_ERR_SIZE;
  if (splits > 1 && (!partials || !counters || lb_attention_decode_scratch(n_seqs, q_heads, dim, splits) > partial_floats ||
                     (long)n_seqs * kv_heads > n_counters))
    return LB_ERR_SIZE;
  configure_once();
  // two K/V stages (three blocks an SM) exist for the served head size with at most 8 heads per KV head
  const bool two_stages = stages == 2 && dim == 128 && q_heads / kv_heads <= 8;
  const size_t smem = decode_smem(dim, two_stages ? 2 : 3);
  if ((3 * (size_t)splits + 1) * (q_heads / kv_heads) * sizeof(float) > smem) return LB_ERR_SIZE;   // merge factors
  const float scale_log2 = scale * 1.4426950408889634f;
  const int chunk_shift = (dim >> 3) <= THREADS ? exact_log2(dim >> 3) : -1, page_shift = exact_log2(page_tokens);
  dim3 grid(n_seqs, kv_heads, splits);
  int code;
  if (two_stages) {
    if (decode_cluster_fits(dim, q_heads / kv_heads, splits, smem))
      code = lb_launch_cluster(attention_decode_kernel<128, true, false, true, 2>, grid, dim3(THREADS), smem, stream, grid.z,
                               (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, block_table, table_width,
                               cu_q, ctx_len, seq_list, q_heads, kv_heads, dim, page_tokens, scale_log2, window, splits,
                               (float*)nullptr, (unsigned*)nullptr, chunk_shift, page_shift);
    else
      code = lb_launch(attention_decode_kernel<128, true, false, false, 2>, grid, dim3(THREADS), smem, stream, (const bf16*)q,
                       (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, block_table, table_width, cu_q, ctx_len, seq_list,
                       q_heads, kv_heads, dim, page_tokens, scale_log2, window, splits, partials, counters, chunk_shift,
                       page_shift);
  } else if (decode_cluster_fits(dim, q_heads / kv_heads, splits, smem))
    code = launch_decode_cluster(q_heads / kv_heads, grid, smem, stream, (const bf16*)q, (const bf16*)k_pool,
                                 (const bf16*)v_pool, (bf16*)out, block_table, table_width, cu_q, ctx_len, seq_list,
                                 q_heads, kv_heads, dim, page_tokens, scale_log2, window, splits, (float*)nullptr,
                                 (unsigned*)nullptr, chunk_shift, page_shift);
  else
    code = launch_decode(dim, q_heads / kv_heads, grid, smem, stream, (const bf16*)q, (const bf16*)k_pool,
                         (const bf16*)v_pool, (bf16*)out, block_table, table_width, cu_q, ctx_len, seq_list,
                         q_heads, kv_heads, dim, page_tokens, scale_log2, window, splits, partials, counters,
                         chunk_shift, page_shift);
  return code ? code : lb_last_error();
}
