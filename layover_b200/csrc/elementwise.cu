// Row-wise kernels of the decoder: embedding gather, (residual add +) RMSNorm, per-head
// QK-norm + rotary embedding + KV page write, SwiGLU. Each is templated on the storage type
// (float for the true 32-bit path, bf16 for serving); all arithmetic is in 32-bit floats and
// the bf16 instantiation rounds where the reference's bf16 tensors round.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// x[t, :] = table[id, :]   (layover/model.py:219,247: no scaling). The id is ids[t], or, where
// token_src[t] >= 0, the last token in record token_src[t] of the per-request records: a step may
// be launched before the host has read the token that the step before it sampled.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ token_src,
                             const int* __restrict__ records, const T* __restrict__ table, T* __restrict__ x,
                             int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  int id = ids[blockIdx.x];
  if (token_src && records) {
    const int slot = token_src[blockIdx.x];
    if (slot >= 0) id = records[(size_t)slot * LB_RECORD_WORDS + LB_RECORD_LAST_TOKEN];
  }
  id = min(max(id, 0), vocab - 1);    // a record that was never sampled into cannot index outside the table
  const T* src = table + (size_t)id * hidden;
  T* dst = x + (size_t)blockIdx.x * hidden;
  if (sizeof(T) * hidden % 16 == 0 && ((uintptr_t)table % 16 == 0) && ((uintptr_t)x % 16 == 0)) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const int n = (int)(sizeof(T) * hidden / 16);
    for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

LB_EXPORT int lb_embed(int dtype, const int* ids, const int* token_src, const int* records, const void* table, void* x,
                       int tokens, int hidden, int vocab, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (vocab <= 0) return LB_ERR_SIZE;
  if (dtype == LB_F32)
    lb_launch(embed_kernel<float>, tokens, 256, 0, stream, ids, token_src, records, (const float*)table, (float*)x, hidden,
              vocab);
  else if (dtype == LB_BF16)
    lb_launch(embed_kernel<bf16>, tokens, 256, 0, stream, ids, token_src, records, (const bf16*)table, (bf16*)x, hidden,
              vocab);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// ---------------------------------------------------------------- add + RMSNorm
// v = x[row] + delta[row] (sum in 32-bit, rounded to T once; written back to x unless rows are
// picked), out = weight * round_T(v * rsqrt(mean(v^2) + eps))   (layover/model.py:31-36,165-166)
// With `rows`, output row r reads source row rows[r] and x is not written (final norm of the
// wanted rows only). The norm weight is always 32-bit.
// eight (bf16) or four (float) elements per 16-byte access
template <typename T> struct Pack;
template <> struct Pack<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Pack<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pair = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
      v[2 * i] = __low2float(pair);
      v[2 * i + 1] = __high2float(pair);
    }
  }
  static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T, bool VEC>
__global__ void add_rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ weight,
                                   T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  extern __shared__ float row_vals[];  // hidden floats + 33 for the reduction
  pdl_launch_dependents();
  pdl_wait();
  float* scratch = row_vals + hidden;
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  T* xr = x + src * hidden;
  const T* dr = delta ? delta + src * hidden : nullptr;
  float ss = 0.f;
  if (VEC) {
    constexpr int N = Pack<T>::N;
    for (int i = threadIdx.x * N; i < hidden; i += blockDim.x * N) {
      float v[N];
      Pack<T>::load(xr + i, v);
      if (dr) {
        float d[N];
        Pack<T>::load(dr + i, d);
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = Elem<T>::round(v[j] + d[j]);
        if (!rows) Pack<T>::store(xr + i, v);
      }
#pragma unroll
      for (int j = 0; j < N; ++j) { row_vals[i + j] = v[j]; ss += v[j] * v[j]; }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = Elem<T>::load(xr + i);
      if (dr) {
        v = Elem<T>::round(v + Elem<T>::load(dr + i));
        if (!rows) Elem<T>::store(xr + i, v);
      }
      row_vals[i] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)blockIdx.x * hidden;
  if (VEC) {
    constexpr int N = Pack<T>::N;
    for (int i = threadIdx.x * N; i < hidden; i += blockDim.x * N) {
      float v[N];
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = weight[i + j] * Elem<T>::round(row_vals[i + j] * inv);
      Pack<T>::store(o + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      Elem<T>::store(o + i, weight[i] * Elem<T>::round(row_vals[i] * inv));
  }
}

// The same for many rows whose width is exactly one 16-byte piece per thread: a block takes RPB rows
// at once, issues the loads of all of them before any arithmetic and keeps the values in registers.
// Every row's sums are taken in the order of the kernel above, so the results are the same bits.
template <typename T, int RPB>
__global__ void add_rmsnorm_rows_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ weight,
                                        T* __restrict__ out, int n_rows, int hidden, float eps) {
  constexpr int N = Pack<T>::N;
  __shared__ float scratch[RPB][33];
  pdl_launch_dependents();
  const int i = threadIdx.x * N, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float w[N];
#pragma unroll
  for (int j = 0; j < N; j += 4) Pack<float>::load(weight + i + j, *reinterpret_cast<float(*)[4]>(&w[j]));   // weights: no kernel writes them
  pdl_wait();
  float v[RPB][N], d[RPB][N], ss[RPB];
#pragma unroll
  for (int r = 0; r < RPB; ++r) {
    const size_t row = (size_t)blockIdx.x * RPB + r;
#pragma unroll
    for (int j = 0; j < N; ++j) v[r][j] = d[r][j] = 0.f;
    if (row < (size_t)n_rows) {
      Pack<T>::load(x + row * hidden + i, v[r]);
      if (delta) Pack<T>::load(delta + row * hidden + i, d[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < RPB; ++r) {
    const size_t row = (size_t)blockIdx.x * RPB + r;
    if (delta) {
#pragma unroll
      for (int j = 0; j < N; ++j) v[r][j] = Elem<T>::round(v[r][j] + d[r][j]);
      if (row < (size_t)n_rows) Pack<T>::store(x + row * hidden + i, v[r]);
    }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) sum += v[r][j] * v[r][j];
    sum = warp_sum(sum);
    if (lane == 0) scratch[r][warp] = sum;
  }
  __syncthreads();
  if (threadIdx.x < RPB) {
    float total = 0.f;
    for (int k = 0; k < nwarps; ++k) total += scratch[threadIdx.x][k];
    scratch[threadIdx.x][32] = total;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < RPB; ++r) {
    const size_t row = (size_t)blockIdx.x * RPB + r;
    ss[r] = scratch[r][32];
    const float inv = 1.0f / sqrtf(ss[r] / (float)hidden + eps);
#pragma unroll
    for (int j = 0; j < N; ++j) v[r][j] = w[j] * Elem<T>::round(v[r][j] * inv);
    if (row < (size_t)n_rows) Pack<T>::store(out + row * hidden + i, v[r]);
  }
}

template <typename T>
static int launch_add_rmsnorm(void* x, const void* delta, const float* weight, void* out, const int* rows, int n_rows,
                              int hidden, float eps, size_t smem, cudaStream_t stream) {
  constexpr int N = Pack<T>::N;
  const bool vec = hidden % N == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                   (!delta || (uintptr_t)delta % 16 == 0);
  // the sum's order depends on the block size only, and that depends on the width only
  int threads = vec ? ((hidden / N + 31) / 32) * 32 : (hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128));
  if (threads > 512) threads = 512;
  if (threads < 32) threads = 32;
  if (vec && !rows && n_rows >= 256 && hidden == threads * N && (uintptr_t)weight % 16 == 0) {
    constexpr int RPB = 2;
    lb_launch(add_rmsnorm_rows_kernel<T, RPB>, (n_rows + RPB - 1) / RPB, threads, 0, stream, (T*)x, (const T*)delta, weight,
              (T*)out, n_rows, hidden, eps);
    return lb_last_error();
  }
  if (vec) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lb_launch(add_rmsnorm_kernel<T, true>, n_rows, threads, smem, stream, (T*)x, (const T*)delta, weight, (T*)out, rows,
              hidden, eps);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lb_launch(add_rmsnorm_kernel<T, false>, n_rows, threads, smem, stream, (T*)x, (const T*)delta, weight, (T*)out, rows,
              hidden, eps);
  }
  return lb_last_error();
}

LB_EXPORT int lb_add_rmsnorm(int dtype, void* x, const void* delta, const float* weight, void* out,
                             const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  if (smem > 200 * 1024) return LB_ERR_SIZE;
  if (dtype == LB_F32) return launch_add_rmsnorm<float>(x, delta, weight, out, rows, n_rows, hidden, eps, smem, stream);
  if (dtype == LB_BF16) return launch_add_rmsnorm<bf16>(x, delta, weight, out, rows, n_rows, hidden, eps, smem, stream);
  return LB_ERR_DTYPE;
}

// ---------------------------------------------------------------- rotary tables
// table[t][0][i] = cos(pos_t * inv_freq[i]), table[t][1][i] = sin(...), 32-bit (layover/model.py:193-197).
// Made once per step and read by every layer, as the reference makes its tables once per call.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ table, int tokens, int n_freq) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * n_freq) return;
  const int t = idx / n_freq, i = idx - t * n_freq;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
  table[((size_t)t * 2) * n_freq + i] = cs;
  table[((size_t)t * 2 + 1) * n_freq + i] = sn;
}

LB_EXPORT int lb_rope_table(const int* positions, const float* inv_freq, float* table, int tokens, int n_freq,
                            cudaStream_t stream) {
  const int total = tokens * n_freq;
  if (total <= 0) return 0;
  lb_launch(rope_table_kernel, (total + 255) / 256, 256, 0, stream, positions, inv_freq, table, tokens, n_freq);
  return lb_last_error();
}

// ---------------------------------------------------------------- QK-norm + rotary + KV write
// Over the (token, head) items of the fused projection row [q heads | k heads | v heads] x dim
// (dim a multiple of 16; rows, outputs and pages 16-byte aligned).
//   q, k: per-head RMSNorm over dim (weight shared by the heads, layover/model.py:124-125), then
//         x*cos + rotate_half(x)*sin with cos/sin from the step's table, rounded to T
//         (layover/model.py:100-102,127-128,193-197); dims >= 2*n_freq pass through unrotated.
//   q is written to q_out [tokens, q_heads, dim]; k and v go to their page:
//         pool[(page * kv_heads + head) * page_tokens + slot][dim], page*page_tokens+slot = slot_map[t]
//         (layover/model.py:133,139-140).
// Null norm weights skip the norm, a null table skips the rotation, null pools skip the write
// (then k is written back in place into the projection row, for a position encoding that runs
// as a separate step), a null q_out skips the q heads (the pass that only writes pages).
// A group of `lanes` lanes (a power of two) serves ROUNDS (1 or 2) consecutive heads of ONE token
// (ROUNDS divides the number of heads), each lane one 16-byte piece of each half of a head; a warp serves
// 32 / lanes such groups. The token's cos/sin pieces are read once for all the group's heads, and
// the loads of all rounds are issued before any arithmetic, so that enough bytes are in flight.
template <typename T, int ROUNDS>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, const float* __restrict__ q_norm_w,
                                       const float* __restrict__ k_norm_w, const float* __restrict__ rope_table,
                                       const int* __restrict__ slot_map,
                                       int tokens, int q_heads, int kv_heads, int dim, int n_freq, int page_tokens,
                                       float eps, int lanes) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int N = Pack<T>::N;
  const int heads = q_heads + 2 * kv_heads, half = dim >> 1;
  const int per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31, sub = lane / lanes, i0 = (lane % lanes) * N;
  const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long total = (long)tokens * heads;
  const long first = (warp * per_warp + sub) * ROUNDS;      // this group's heads: first .. first + ROUNDS - 1
  const bool mine = i0 < half, live = first < total;        // heads % ROUNDS == 0: a group is all live or all not
  const int t = live ? (int)(first / heads) : 0, h0 = live ? (int)(first % heads) : 0;

  float lo[ROUNDS][N], hi[ROUNDS][N], cs[N], sn[N];
  const bool rotate = rope_table && i0 + N <= n_freq;    // n_freq = half whenever a table is given
#pragma unroll
  for (int j = 0; j < N; ++j) { cs[j] = 1.f; sn[j] = 0.f; }
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
#pragma unroll
    for (int j = 0; j < N; ++j) lo[r][j] = hi[r][j] = 0.f;
    if (live && mine) {
      const T* src = qkv + (size_t)(first + r) * dim;
      Pack<T>::load(src + i0, lo[r]);
      Pack<T>::load(src + i0 + half, hi[r]);
    }
  }
  if (live && mine && rotate && h0 < q_heads + kv_heads) {     // the table's values travel with the data
    const float* cos_row = rope_table + ((size_t)t * 2) * n_freq + i0;
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      float c4[4], s4[4];
      Pack<float>::load(cos_row + j, c4);
      Pack<float>::load(cos_row + n_freq + j, s4);
#pragma unroll
      for (int e = 0; e < 4; ++e) { cs[j + e] = Elem<T>::round(c4[e]); sn[j + e] = Elem<T>::round(s4[e]); }
    }
  }
  int slot = 0;
  if (live && h0 + ROUNDS > q_heads && (k_pool || v_pool)) slot = slot_map[t];
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const int h = h0 + r;
    const bool is_q = h < q_heads, is_k = !is_q && h < q_heads + kv_heads;
    T* dst = nullptr;
    if (live) {
      if (is_q) {
        dst = q_out ? q_out + ((size_t)t * q_heads + h) * dim : nullptr;   // null: a pass that only writes pages
      } else {
        T* pool = is_k ? k_pool : v_pool;
        if (pool) {
          const int kvh = is_k ? h - q_heads : h - q_heads - kv_heads;
          const size_t page = slot / page_tokens, within = slot % page_tokens;
          dst = pool + ((page * kv_heads + kvh) * page_tokens + within) * dim;
        } else {
          dst = is_k ? qkv + (size_t)(first + r) * dim : nullptr;          // k goes back in place, v stays
        }
      }
    }
    const float* w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) ss += lb_square_pair(lo[r][j], hi[r][j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      if (o < lanes) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // whole groups agree, every lane joins
    if (!dst || !mine) continue;
    if (w) {
      const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        lo[r][j] = Elem<T>::round(w[i0 + j] * Elem<T>::round(lo[r][j] * inv));
        hi[r][j] = Elem<T>::round(w[i0 + j + half] * Elem<T>::round(hi[r][j] * inv));
      }
    }
    if (rotate && (is_q || is_k)) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        // rotate_half(x) = (-hi, lo): each product and the sum round to T
        const float a = Elem<T>::round(Elem<T>::round(lo[r][j] * cs[j]) + Elem<T>::round(-hi[r][j] * sn[j]));
        const float b = Elem<T>::round(Elem<T>::round(hi[r][j] * cs[j]) + Elem<T>::round(lo[r][j] * sn[j]));
        lo[r][j] = a;
        hi[r][j] = b;
      }
    }
    Pack<T>::store(dst + i0, lo[r]);
    Pack<T>::store(dst + i0 + half, hi[r]);
  }
}

template <typename T, int ROUNDS>
static void launch_qk_norm_rope_kv(void* qkv, void* q_out, void* k_pool, void* v_pool, const float* q_norm_w,
                                   const float* k_norm_w, const float* rope_table, const int* slot_map, int tokens,
                                   int q_heads, int kv_heads, int dim, int n_freq, int page_tokens, float eps, int lanes,
                                   cudaStream_t stream) {
  const long groups = (long)tokens * (q_heads + 2 * kv_heads) / ROUNDS;
  const int per_warp = 32 / lanes, threads = 128;
  const long warps = (groups + per_warp - 1) / per_warp;
  const long blocks = (warps * 32 + threads - 1) / threads;
  lb_launch(qk_norm_rope_kv_kernel<T, ROUNDS>, (unsigned)blocks, threads, 0, stream, (T*)qkv, (T*)q_out, (T*)k_pool,
            (T*)v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads, kv_heads, dim, n_freq, page_tokens, eps,
            lanes);
}

template <typename T>
static void dispatch_qk_norm_rope_kv(void* qkv, void* q_out, void* k_pool, void* v_pool, const float* q_norm_w,
                                     const float* k_norm_w, const float* rope_table, const int* slot_map, int tokens,
                                     int q_heads, int kv_heads, int dim, int n_freq, int page_tokens, float eps, int lanes,
                                     cudaStream_t stream) {
  const int heads = q_heads + 2 * kv_heads;
  // two heads share the read of the token's cos/sin row; four measured slower (29 against 23 us for
  // 2,048 tokens of 48 heads: 114 registers a thread leave too few warps in flight)
  if (heads % 2 == 0)
    launch_qk_norm_rope_kv<T, 2>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                 kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
  else
    launch_qk_norm_rope_kv<T, 1>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                 kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
}

LB_EXPORT int lb_qk_norm_rope_kv(int dtype, void* qkv, void* q_out, void* k_pool, void* v_pool,
                                 const float* q_norm_w, const float* k_norm_w, const float* rope_table,
                                 const int* slot_map, int tokens, int q_heads, int kv_heads, int dim, int n_freq,
                                 int page_tokens, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dim % 16 || dim > 512 || 2 * n_freq > dim) return LB_ERR_SIZE;   // one 16-byte piece of each half per lane
  // a rotation pairs i with i + dim/2 only when the rotary part spans the whole head
  if (rope_table && 2 * n_freq != dim) return LB_ERR_SIZE;
  const int piece = dtype == LB_BF16 ? 8 : 4;               // elements in 16 bytes
  int lanes = 1;
  while (lanes * piece * 2 < dim) lanes *= 2;
  if (dtype == LB_F32)
    dispatch_qk_norm_rope_kv<float>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                    kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
  else if (dtype == LB_BF16)
    dispatch_qk_norm_rope_kv<bf16>(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, rope_table, slot_map, tokens, q_heads,
                                   kv_heads, dim, n_freq, page_tokens, eps, lanes, stream);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

// ---------------------------------------------------------------- SwiGLU
// out[t, j] = silu(gu[t, j]) * gu[t, inter + j], silu(z) = z / (1 + exp(-z)); silu and the
// product each round to T (layover/model.py:152-153).
// `block` 0: the row is [all gates | all ups]. `block` b > 0: gates and ups alternate in blocks of b
// features ([b gates | b ups | b gates | ...]), the layout of the products' fused epilogue.
template <typename T, bool VEC>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long total, int inter, int block) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int N = VEC ? Pack<T>::N : 1;
  const long idx = ((long)blockIdx.x * blockDim.x + threadIdx.x) * N;
  if (idx >= total) return;
  const long t = idx / inter;
  const int j = (int)(idx - t * inter);
  const T* gp = gate_up + t * 2 * inter + (block > 0 ? (j / block) * 2 * block + j % block : j);
  const int up_at = block > 0 ? block : inter;
  if (VEC) {
    float g[Pack<T>::N], u[Pack<T>::N];
    Pack<T>::load(gp, g);
    Pack<T>::load(gp + up_at, u);
#pragma unroll
    for (int i = 0; i < Pack<T>::N; ++i) g[i] = Elem<T>::round(g[i] / (1.0f + expf(-g[i]))) * u[i];
    Pack<T>::store(out + idx, g);
  } else {
    const float g = Elem<T>::load(gp), u = Elem<T>::load(gp + up_at);
    Elem<T>::store(out + idx, Elem<T>::round(g / (1.0f + expf(-g))) * u);
  }
}

template <typename T>
static int launch_swiglu(const void* gate_up, void* out, long total, int inter, int block, cudaStream_t stream) {
  constexpr int N = Pack<T>::N;
  const bool vec = inter % N == 0 && (block == 0 || block % N == 0) && (uintptr_t)gate_up % 16 == 0 &&
                   (uintptr_t)out % 16 == 0;
  const int threads = 256;
  const long work = vec ? total / N : total;
  const unsigned blocks = (unsigned)((work + threads - 1) / threads);
  if (vec) lb_launch(swiglu_kernel<T, true>, blocks, threads, 0, stream, (const T*)gate_up, (T*)out, total, inter, block);
  else lb_launch(swiglu_kernel<T, false>, blocks, threads, 0, stream, (const T*)gate_up, (T*)out, total, inter, block);
  return lb_last_error();
}

LB_EXPORT int lb_swiglu(int dtype, const void* gate_up, void* out, int tokens, int inter, int block,
                        cudaStream_t stream) {
  const long total = (long)tokens * inter;
  if (total <= 0) return 0;
  if (block < 0 || (block > 0 && inter % block)) return LB_ERR_SIZE;
  if (dtype == LB_F32) return launch_swiglu<float>(gate_up, out, total, inter, block, stream);
  if (dtype == LB_BF16) return launch_swiglu<bf16>(gate_up, out, total, inter, block, stream);
  return LB_ERR_DTYPE;
}
