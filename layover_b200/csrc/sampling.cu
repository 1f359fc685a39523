// Greedy and temperature sampling over 32-bit logits [rows, vocab].
//
// Greedy is the first index of the maximum (layover/engine.py:139-141,187). The reference
// accepts a temperature and ignores it (layover/server.py:13-14); here a temperature T > 0
// draws from softmax(logits / T) by the Gumbel-max rule
//     token = argmax_v ( logits[v] / T - log(-log(u_v)) ),
// with u_v from Philox-4x32-10 keyed by the request's seed and counted by (v / 4, number of
// tokens the request has sampled so far): a draw depends on nothing but the request's own
// seed, step and logits, so it is the same in any batch.
#include <math.h>

#include "common.cuh"

namespace {
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
  c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

constexpr int THREADS = 1024;

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long row_stride, int vocab, const float* __restrict__ temperature,
              const uint32_t* __restrict__ seed_lo, const uint32_t* __restrict__ seed_hi,
              const uint32_t* __restrict__ step, int* __restrict__ tokens) {
  __shared__ float best_val[THREADS / 32];
  __shared__ int best_idx[THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const float* lg = logits + (long)row * row_stride;
  const float temp = temperature ? temperature[row] : 0.f;
  float best = -INFINITY;
  int arg = 0x7fffffff;
  const int blocks = (vocab + 3) / 4;
  for (int b = threadIdx.x; b < blocks; b += THREADS) {
    float noise[4] = {0.f, 0.f, 0.f, 0.f};
    if (temp > 0.f) {
      uint32_t c[4] = {(uint32_t)b, step[row], 0u, 0u};
      philox4x32_10(c, seed_lo[row], seed_hi[row]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float u = ((float)(c[j] >> 8) + 0.5f) * 5.9604644775390625e-08f;  // 2^-24
        noise[j] = -logf(-logf(u));
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = 4 * b + j;
      if (v < vocab) {
        const float val = temp > 0.f ? lg[v] / temp + noise[j] : lg[v];
        if (val > best || (val == best && v < arg)) { best = val; arg = v; }
      }
    }
  }
  // lowest index among equal maxima, first in the warp, then over the warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
  }
  if ((threadIdx.x & 31) == 0) { best_val[threadIdx.x >> 5] = best; best_idx[threadIdx.x >> 5] = arg; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < THREADS / 32; ++w)
      if (best_val[w] > best || (best_val[w] == best && best_idx[w] < arg)) { best = best_val[w]; arg = best_idx[w]; }
    // a row without any finite maximum (all NaN) still yields a token inside the vocabulary
    tokens[row] = arg == 0x7fffffff ? 0 : arg;
  }
}
}  // namespace

LB_EXPORT int lb_sample(const float* logits, long row_stride, int rows, int vocab, const float* temperature,
                        const uint32_t* seed_lo, const uint32_t* seed_hi, const uint32_t* step, int* tokens,
                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return LB_ERR_SIZE;
  lb_launch(sample_kernel, rows, THREADS, 0, stream, logits, row_stride, vocab, temperature, seed_lo, seed_hi, step, tokens);
  return lb_last_error();
}
