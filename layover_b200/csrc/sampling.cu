// Greedy and temperature sampling over 32-bit logits [rows, vocab].
//
// Greedy is the first index of the maximum (layover/engine.py:139-141,187). The reference
// accepts a temperature and ignores it (layover/server.py:13-14); here a temperature T > 0
// draws from softmax(logits / T) by the Gumbel-max rule
//     token = argmax_v ( logits[v] / T - log(-log(u_v)) ),
// with u_v from Philox-4x32-10 keyed by the request's seed and counted by (v / 4, number of
// tokens the request has sampled so far): a draw depends on nothing but the request's own
// seed, step and logits, so it is the same in any batch. Seed, counter and temperature live in
// the request's record on the device (written once when it is admitted), so a step uploads
// nothing for sampling.
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

// One block per row of logits. What a row's request wants is in its record (common.cuh): with
// `records`, row r belongs to the request in slot row_slots[r]; the kernel reads temperature, seed
// and counter there, stores the chosen token as the request's last token, bumps the counter and sets
// the request's position to positions[logit_rows[r]] + 2 (the tokens it holds once the chosen token
// is counted too). Without `records` every row is greedy and nothing but `tokens` is written.
// Block 0 also copies the error words of other kernel libraries (`status_words`: device addresses)
// behind the tokens, tokens[rows + i], so that the host learns of a wait that ran out with the
// tokens it reads anyway.
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long row_stride, int rows, int vocab, int* __restrict__ records,
              const int* __restrict__ row_slots, const int* __restrict__ positions, const int* __restrict__ logit_rows,
              int* __restrict__ tokens, const unsigned long long* __restrict__ status_words, int n_status) {
  __shared__ float best_val[THREADS / 32];
  __shared__ int best_idx[THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  if (row == 0 && threadIdx.x < n_status) {
    const int* word = reinterpret_cast<const int*>(status_words[threadIdx.x]);
    tokens[rows + threadIdx.x] = word ? *reinterpret_cast<const volatile int*>(word) : 0;
  }
  const float* lg = logits + (long)row * row_stride;
  int* record = records ? records + (size_t)row_slots[row] * LB_RECORD_WORDS : nullptr;
  const float temp = record ? __int_as_float(record[LB_RECORD_TEMPERATURE]) : 0.f;
  const uint32_t seed_lo = record ? (uint32_t)record[LB_RECORD_SEED_LO] : 0u;
  const uint32_t seed_hi = record ? (uint32_t)record[LB_RECORD_SEED_HI] : 0u;
  const uint32_t step = record ? (uint32_t)record[LB_RECORD_COUNT] : 0u;
  float best = -INFINITY;
  int arg = 0x7fffffff;
  const int blocks = (vocab + 3) / 4;
  for (int b = threadIdx.x; b < blocks; b += THREADS) {
    float noise[4] = {0.f, 0.f, 0.f, 0.f};
    if (temp > 0.f) {
      uint32_t c[4] = {(uint32_t)b, step, 0u, 0u};
      philox4x32_10(c, seed_lo, seed_hi);
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
    const int token = arg == 0x7fffffff ? 0 : arg;
    tokens[row] = token;
    if (record) {
      record[LB_RECORD_LAST_TOKEN] = token;
      record[LB_RECORD_COUNT] = (int)(step + 1u);
      if (positions && logit_rows) record[LB_RECORD_POSITION] = positions[logit_rows[row]] + 2;
    }
  }
}
}  // namespace

// tokens must hold rows + n_status ints.
LB_EXPORT int lb_sample(const float* logits, long row_stride, int rows, int vocab, int* records, const int* row_slots,
                        const int* positions, const int* logit_rows, int* tokens,
                        const unsigned long long* status_words, int n_status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || n_status < 0 || n_status > THREADS || (records && !row_slots)) return LB_ERR_SIZE;
  lb_launch(sample_kernel, rows, THREADS, 0, stream, logits, row_stride, rows, vocab, records, row_slots, positions,
            logit_rows, tokens, status_words, n_status);
  return lb_last_error();
}
