// The allocation-free variant of the split-K decode attention (see decode_attention_static.h for
// who needs it, its limits and its rules). The kernel is the very one the regular entry point
// launches; only the home of the scratch memory differs: a file-scope array of this library.
#include "decode_attention_static.h"

#include "attention_mma.cu"   // the kernels (file-local there, so this library gets its own copy)

// Counters first (zero between calls), partial outputs after them.
static __device__ __align__(256) unsigned char g_static_scratch[LB_STATIC_SCRATCH_BYTES];

namespace {

constexpr int MAX_DEVICES = 64;
void* g_scratch_address[MAX_DEVICES] = {};   // device address of the array, per device, once known

// In host code `g_static_scratch` names a host-side stand-in, not device memory: handing it to a
// kernel would fault or silently use the wrong bytes. The device address comes from the runtime,
// once per device, with that device current.
int scratch_for_current_device(void** address) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return LB_STATIC_ERR_SETUP;
  if (!g_scratch_address[device]) {
    void* found = nullptr;
    if (cudaGetSymbolAddress(&found, g_static_scratch) != cudaSuccess || !found) {
      cudaGetLastError();
      return LB_STATIC_ERR_SETUP;
    }
    configure_once();   // raises the kernels' shared-memory limit; allocates nothing
    g_scratch_address[device] = found;
  }
  *address = g_scratch_address[device];
  return 0;
}
}  // namespace

extern "C" __attribute__((visibility("default")))
int lb_attention_decode_bf16_static(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    const int* block_table, int table_width, const int* cu_q, const int* ctx_len,
                                    int n_seqs, int q_heads, int kv_heads, int dim, int page_tokens, float scale,
                                    int window, int splits, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (dim <= 0 || dim % 16 || dim > 256 || kv_heads <= 0 || q_heads % kv_heads || q_heads / kv_heads > 16 ||
      kv_heads > 65535 || splits < 1 || splits > 65535 || page_tokens <= 0)
    return LB_STATIC_ERR_SHAPE;
  const size_t smem = decode_smem(dim);
  if ((3 * (size_t)splits + 1) * (q_heads / kv_heads) * sizeof(float) > smem) return LB_STATIC_ERR_SHAPE;
  const long counters_needed = (long)n_seqs * kv_heads;
  const long partial_floats = splits > 1 ? (long)n_seqs * q_heads * splits * (dim + 2) : 0;
  if (counters_needed > LB_STATIC_MAX_COUNTERS || partial_floats > LB_STATIC_MAX_PARTIAL_FLOATS)
    return LB_STATIC_ERR_TOO_LARGE;

  void* base = nullptr;
  const int setup = scratch_for_current_device(&base);
  if (setup) return setup;
  unsigned* counters = static_cast<unsigned*>(base);
  float* partials = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + LB_STATIC_MAX_COUNTERS * 4);
  if (splits > 1) {
    // the array keeps the last call's contents; the counters of this call must start at zero
    const cudaError_t cleared = cudaMemsetAsync(counters, 0, (size_t)counters_needed * sizeof(unsigned), stream);
    if (cleared != cudaSuccess) return (int)cleared;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  const int chunk_shift = (dim >> 3) <= THREADS ? exact_log2(dim >> 3) : -1, page_shift = exact_log2(page_tokens);
  dim3 grid(n_seqs, kv_heads, splits);
  const int code = launch_decode(dim, q_heads / kv_heads, grid, smem, stream, (const bf16*)q, (const bf16*)k_pool,
                                 (const bf16*)v_pool, (bf16*)out, block_table, table_width, cu_q, ctx_len,
                                 (const int*)nullptr, q_heads, kv_heads, dim, page_tokens, scale_log2, window, splits, partials,
                                 counters, chunk_shift, page_shift);
  return code ? code : lb_last_error();
}

extern "C" __attribute__((visibility("default")))
const char* lb_attention_decode_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case LB_STATIC_ERR_TOO_LARGE:
      return "the batch needs more split-K scratch than the library's static array holds "
             "(n_seqs * kv_heads <= 4096 and n_seqs * q_heads * splits * (dim + 2) <= 1048576)";
    case LB_STATIC_ERR_SETUP: return "the device address of the static scratch array could not be obtained";
    case LB_STATIC_ERR_SHAPE: return "head size, head counts or number of splits outside what the kernel takes";
    default: return code > 0 ? "a CUDA error from the launch (the value is a cudaError_t)" : "unknown error";
  }
}
