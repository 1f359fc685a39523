// A toy mixer's own kernel, outside the package: per request a running mean of its inputs.
//
// state[slot] holds hidden sums and, last, the number of tokens seen so far. For every sequence s of
// the batch (rows cu_q[s] .. cu_q[s + 1] of h, state slot slots[s]) and every channel c, the tokens are
// taken in order: sum += h[t][c], out[t][c] = sum / count. One block per sequence, one thread per
// channel (strided), so a request's tokens are a scan and chunk boundaries are state hand-offs.
#include <cuda_runtime.h>

namespace {
__global__ void running_mean_kernel(const float* __restrict__ h, float* __restrict__ out, float* __restrict__ state,
                                    const int* __restrict__ cu_q, const int* __restrict__ slots, int hidden) {
  const int seq = blockIdx.x, first = cu_q[seq], last = cu_q[seq + 1];
  float* mine = state + (size_t)slots[seq] * (hidden + 1);
  const float seen = mine[hidden];
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float sum = mine[c];
    for (int t = first; t < last; ++t) {
      sum += h[(size_t)t * hidden + c];
      out[(size_t)t * hidden + c] = sum / (seen + (float)(t - first + 1));
    }
    mine[c] = sum;
  }
  __syncthreads();      // every thread has read the old count
  if (threadIdx.x == 0) mine[hidden] = seen + (float)(last - first);
}
}  // namespace

extern "C" __attribute__((visibility("default")))
int toy_running_mean(const float* h, float* out, float* state, const int* cu_q, const int* slots, int n_seqs, int hidden,
                     cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  running_mean_kernel<<<n_seqs, 128, 0, stream>>>(h, out, state, cu_q, slots, hidden);
  return (int)cudaGetLastError();
}
