// Paged grouped-query attention over the block table, 32-bit arithmetic throughout, one kernel
// for every segment length: a whole prompt, a portion of one, or a single decoded token.
//
//   s_j = (q . K_j) / sqrt(dim)      for keys j <= p and (window == 0 or p - j < window)
//   o   = sum_j softmax(s)_j V_j     (layover/model.py:59,90-96; layover/kernels/triton_decode.py:89-119)
//
// where p is the query's absolute position. Keys are walked in tiles of 32 aligned to absolute
// positions (tile i holds keys [32 i, 32 i + 32)), each score is one sequential dot product and
// the running maximum / sum follow the same recurrence for every row, so a row's result does
// not depend on how the tokens were cut into steps or on which other rows share its block.
// Keys outside [first needed key, context length) are never used: their scores are replaced,
// not multiplied, and their values are read as zero, so stale or non-finite contents of a page
// cannot leak.
//
// Work is a list of tiles made on the host: tile w covers queries [tile_q0[w], +BQ) of sequence
// tile_seq[w]. Grid = (tiles, query heads). Query t of sequence s is row cu_q[s] + t of q and
// out, at absolute position ctx_len[s] - q_len(s) + t.
#include <math.h>

#include "common.cuh"

namespace {
constexpr int BQ = 16;      // queries per block
constexpr int BKEYS = 32;   // keys per tile (one per lane)
constexpr int WARPS = 4;
constexpr int ROWS_PER_WARP = BQ / WARPS;
constexpr int MAX_DIM = 256;
constexpr int ACC_PER_LANE = MAX_DIM / 32;

// four neighbouring elements with one load (the head size is a multiple of 4 and rows are 16-byte aligned)
template <typename T> struct Quad;
template <> struct Quad<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Quad<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
};

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                            T* __restrict__ out, const int* __restrict__ block_table, int table_width,
                            const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                            const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, int q_heads,
                            int kv_heads, int dim, int page_tokens, float scale, int window) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  float* q_s = smem;                               // [BQ][dim]
  float* k_s = q_s + BQ * dim;                     // [BKEYS][dim + 1]
  float* v_s = k_s + BKEYS * (dim + 1);            // [BKEYS][dim]

  const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
  const int head = blockIdx.y, kv_head = head / (q_heads / kv_heads);
  const int row0 = cu_q[seq], q_len = cu_q[seq + 1] - row0, ctx = ctx_len[seq];
  const int start = ctx - q_len;                   // absolute position of the sequence's first query here
  const int n_q = min(BQ, q_len - q0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table = block_table + (size_t)seq * table_width;

  for (int i = threadIdx.x; i < n_q * dim; i += blockDim.x) {
    const int r = i / dim, c = i % dim;
    q_s[r * dim + c] = Elem<T>::load(q + ((size_t)(row0 + q0 + r) * q_heads + head) * dim + c);
  }

  const int p_first = start + q0, p_last = start + q0 + n_q - 1;
  const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;  // first key any row here may see
  const int tile_lo = key_lo / BKEYS, tile_hi = p_last / BKEYS;

  float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][ACC_PER_LANE];
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < ACC_PER_LANE; ++c) acc[r][c] = 0.f;
  }

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    __syncthreads();  // the previous tile is no longer read (and q_s is complete)
    const int quads = dim >> 2;
    for (int i = threadIdx.x; i < BKEYS * quads; i += blockDim.x) {
      const int j = i / quads, c = (i - j * quads) << 2;
      const int key = tile * BKEYS + j;
      float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
      if (key >= key_lo && key <= p_last) {
        const size_t page = (size_t)table[key / page_tokens];
        const size_t at = ((page * kv_heads + kv_head) * page_tokens + key % page_tokens) * dim + c;
        kv = Quad<T>::load(k_pool + at);
        vv = Quad<T>::load(v_pool + at);
      }
      float* kd = k_s + j * (dim + 1) + c;
      kd[0] = kv.x; kd[1] = kv.y; kd[2] = kv.z; kd[3] = kv.w;
      *reinterpret_cast<float4*>(v_s + j * dim + c) = vv;
    }
    __syncthreads();
    const int key = tile * BKEYS + lane;
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) {
      const int row = warp * ROWS_PER_WARP + r;
      if (row >= n_q) continue;  // uniform over the warp
      const int p = p_first + row;
      const bool seen = key <= p && (window <= 0 || p - key < window);
      float s = 0.f;
      const float* qr = q_s + row * dim;
      const float* kr = k_s + lane * (dim + 1);
      for (int c = 0; c < dim; ++c) s = fmaf(qr[c], kr[c], s);
      s = seen ? s * scale : -INFINITY;
      const float tile_max = warp_max(s);
      if (tile_max == -INFINITY) continue;  // nothing of this tile is seen by this row
      const float m_new = fmaxf(m[r], tile_max);
      const float prob = seen ? expf(s - m_new) : 0.f;
      const float alpha = m[r] == -INFINITY ? 0.f : expf(m[r] - m_new);
      l[r] = l[r] * alpha + warp_sum(prob);
      m[r] = m_new;
#pragma unroll
      for (int c = 0; c < ACC_PER_LANE; ++c) acc[r][c] *= alpha;
      for (int j = 0; j < BKEYS; ++j) {
        const float pj = __shfl_sync(0xffffffffu, prob, j);
#pragma unroll
        for (int c = 0; c < ACC_PER_LANE; ++c) {
          const int d = lane + 32 * c;
          if (d < dim) acc[r][c] = fmaf(pj, v_s[j * dim + d], acc[r][c]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    const int row = warp * ROWS_PER_WARP + r;
    if (row >= n_q) continue;
    T* o = out + ((size_t)(row0 + q0 + row) * q_heads + head) * dim;
#pragma unroll
    for (int c = 0; c < ACC_PER_LANE; ++c) {
      const int d = lane + 32 * c;
      if (d < dim) Elem<T>::store(o + d, acc[r][c] / l[r]);
    }
  }
}
}  // namespace

LB_EXPORT int lb_attention_simt_block_queries() { return BQ; }

LB_EXPORT int lb_attention_simt(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                const int* block_table, int table_width, const int* cu_q, const int* ctx_len,
                                const int* tile_seq, const int* tile_q0, int n_tiles, int q_heads, int kv_heads,
                                int dim, int page_tokens, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (dim <= 0 || dim > MAX_DIM || dim % 4 || kv_heads <= 0 || q_heads % kv_heads || q_heads > 65535) return LB_ERR_SIZE;
  const size_t smem = (size_t)(BQ * dim + BKEYS * (dim + 1) + BKEYS * dim) * sizeof(float);
  dim3 grid(n_tiles, q_heads);
  if (dtype == LB_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(paged_attention_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lb_launch(paged_attention_simt_kernel<float>, grid, WARPS * 32, smem, stream, 
        (const float*)q, (const float*)k_pool, (const float*)v_pool, (float*)out, block_table, table_width, cu_q,
        ctx_len, tile_seq, tile_q0, q_heads, kv_heads, dim, page_tokens, scale, window);
  } else if (dtype == LB_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(paged_attention_simt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lb_launch(paged_attention_simt_kernel<bf16>, grid, WARPS * 32, smem, stream, 
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, block_table, table_width, cu_q, ctx_len,
        tile_seq, tile_q0, q_heads, kv_heads, dim, page_tokens, scale, window);
  } else
    return LB_ERR_DTYPE;
  return lb_last_error();
}
