// C[M, N] = A[M, K] * W[N, K]^T with 32-bit FFMA accumulation: the matrix product of the true
// 32-bit path (no tensor cores, no TF32), also instantiated for bf16 operands as the slow
// oracle of the tensor-core kernel. Row strides are given in elements.
//
// Each output element is one sequential sum over k = 0..K-1 in a fixed order, whatever M is
// and wherever the row sits in its tile, so a token's result does not depend on how a batch
// was cut. Any M, N, K >= 1 is accepted; rows whose address and stride allow it are loaded
// four elements at a time.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
};

// loads a [rows_in_tile=64, BK] slab, K-contiguous in memory, into smem transposed [BK][64+4]
template <typename T>
__device__ __forceinline__ void load_slab(const T* __restrict__ base, long ld, int row0, int n_rows, int k0, int K,
                                          bool vec_ok, float (*dst)[BM + 4]) {
  const int r = threadIdx.x >> 2, kk = (threadIdx.x & 3) * 4;
  const int row = row0 + r;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (row < n_rows) {
    const T* p = base + (long)row * ld + k0 + kk;
    if (vec_ok && k0 + kk + 3 < K) {
      Vec4<T>::load(p, v);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (k0 + kk + j < K) v[j] = Elem<T>::load(p + j);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) dst[kk + j][r] = v[j];
}

template <typename TA, typename TC>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                 long lda, long ldw, long ldc, bool vec_a, bool vec_w) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    load_slab<TA>(A, lda, m0, M, k0, K, vec_a, As);
    load_slab<TA>(W, ldw, n0, N, k0, K, vec_w, Ws);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int row = m0 + ty * TM + i;
    if (row >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int col = n0 + tx * TN + j;
      if (col < N) Elem<TC>::store(C + (long)row * ldc + col, acc[i][j]);
    }
  }
}

// The same product for steps of at most 16 tokens: tiles of 16 tokens x 16 weight rows, so that a
// weight matrix of a few thousand rows still gives every SM a block (the 64 x 64 tiles above leave
// most of the GPU idle then and spend 7/8 of their arithmetic on rows that are not there). A thread
// owns one weight row and two tokens; the next slab of 32 k is fetched into registers while the
// current one is used. Every output element is still ONE sequential fused-multiply-add chain over
// k = 0..K-1 starting from zero, so it has the bits the large-tile kernel gives the same token.
constexpr int FT_M = 16, FT_N = 16, FT_K = 32, FT_THREADS = 128;

template <typename T>
__device__ __forceinline__ void fetch_quad(const T* __restrict__ base, long ld, int row, int n_rows, int k, int K, bool vec,
                                           float (&v)[4]) {
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (row >= n_rows) return;
  const T* p = base + (long)row * ld + k;
  if (vec && k + 3 < K) {
    Vec4<T>::load(p, v);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (k + j < K) v[j] = Elem<T>::load(p + j);
  }
}

template <typename TA, typename TC>
__global__ void __launch_bounds__(FT_THREADS)
gemm_simt_fewtoken_kernel(const TA* __restrict__ A, const TA* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                          long lda, long ldw, long ldc, bool vec_a, bool vec_w) {
  __shared__ float As[FT_K][FT_M + 1];
  __shared__ float Ws[FT_K][FT_N + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int n0 = blockIdx.x * FT_N, m0 = blockIdx.y * FT_M;
  const int lr = threadIdx.x >> 3, lk = (threadIdx.x & 7) * 4;      // the row and the four k this thread fetches of a slab
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;           // weight row of the tile, pair of tokens
  float acc[2] = {0.f, 0.f};
  float next_a[4], next_w[4];
  fetch_quad<TA>(A, lda, m0 + lr, M, lk, K, vec_a, next_a);
  fetch_quad<TA>(W, ldw, n0 + lr, N, lk, K, vec_w, next_w);
  for (int k0 = 0; k0 < K; k0 += FT_K) {
#pragma unroll
    for (int j = 0; j < 4; ++j) { As[lk + j][lr] = next_a[j]; Ws[lk + j][lr] = next_w[j]; }
    __syncthreads();
    if (k0 + FT_K < K) {
      fetch_quad<TA>(A, lda, m0 + lr, M, k0 + FT_K + lk, K, vec_a, next_a);
      fetch_quad<TA>(W, ldw, n0 + lr, N, k0 + FT_K + lk, K, vec_w, next_w);
    }
    const int steps = min(FT_K, K - k0);
    if (steps == FT_K) {
#pragma unroll
      for (int k = 0; k < FT_K; ++k) {
        const float w = Ws[k][tx];
        acc[0] = fmaf(As[k][2 * ty], w, acc[0]);
        acc[1] = fmaf(As[k][2 * ty + 1], w, acc[1]);
      }
    } else {
      for (int k = 0; k < steps; ++k) {      // the k beyond K would add exact zeros; they are left out all the same
        const float w = Ws[k][tx];
        acc[0] = fmaf(As[k][2 * ty], w, acc[0]);
        acc[1] = fmaf(As[k][2 * ty + 1], w, acc[1]);
      }
    }
    __syncthreads();
  }
  const int col = n0 + tx;
  if (col < N) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = m0 + 2 * ty + i;
      if (row < M) Elem<TC>::store(C + (long)row * ldc + col, acc[i]);
    }
  }
}

template <typename T> bool vec_ok(const void* p, long ld) {
  return ((uintptr_t)p % (4 * sizeof(T)) == 0) && (ld % 4 == 0);
}
}  // namespace

// in_dtype: type of A and W; out_dtype: type of C (bf16 inputs may write 32-bit floats).
LB_EXPORT int lb_gemm_simt(int in_dtype, int out_dtype, const void* A, const void* W, void* C, int M, int N, int K,
                           long lda, long ldw, long ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return LB_ERR_SIZE;
  if (M <= FT_M) {
    dim3 few((N + FT_N - 1) / FT_N, 1);
    if (in_dtype == LB_F32 && out_dtype == LB_F32)
      lb_launch(gemm_simt_fewtoken_kernel<float, float>, few, FT_THREADS, 0, stream, (const float*)A, (const float*)W, (float*)C,
                M, N, K, lda, ldw, ldc, vec_ok<float>(A, lda), vec_ok<float>(W, ldw));
    else if (in_dtype == LB_BF16 && out_dtype == LB_BF16)
      lb_launch(gemm_simt_fewtoken_kernel<bf16, bf16>, few, FT_THREADS, 0, stream, (const bf16*)A, (const bf16*)W, (bf16*)C, M, N,
                K, lda, ldw, ldc, vec_ok<bf16>(A, lda), vec_ok<bf16>(W, ldw));
    else if (in_dtype == LB_BF16 && out_dtype == LB_F32)
      lb_launch(gemm_simt_fewtoken_kernel<bf16, float>, few, FT_THREADS, 0, stream, (const bf16*)A, (const bf16*)W, (float*)C, M,
                N, K, lda, ldw, ldc, vec_ok<bf16>(A, lda), vec_ok<bf16>(W, ldw));
    else
      return LB_ERR_DTYPE;
    return lb_last_error();
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return LB_ERR_SIZE;
  if (in_dtype == LB_F32 && out_dtype == LB_F32)
    lb_launch(gemm_simt_kernel<float, float>, grid, THREADS, 0, stream, (const float*)A, (const float*)W, (float*)C, M, N, K,
                                                                 lda, ldw, ldc, vec_ok<float>(A, lda),
                                                                 vec_ok<float>(W, ldw));
  else if (in_dtype == LB_BF16 && out_dtype == LB_BF16)
    lb_launch(gemm_simt_kernel<bf16, bf16>, grid, THREADS, 0, stream, (const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda,
                                                               ldw, ldc, vec_ok<bf16>(A, lda), vec_ok<bf16>(W, ldw));
  else if (in_dtype == LB_BF16 && out_dtype == LB_F32)
    lb_launch(gemm_simt_kernel<bf16, float>, grid, THREADS, 0, stream, (const bf16*)A, (const bf16*)W, (float*)C, M, N, K,
                                                                lda, ldw, ldc, vec_ok<bf16>(A, lda),
                                                                vec_ok<bf16>(W, ldw));
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}
