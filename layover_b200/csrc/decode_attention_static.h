// Split-K paged decode attention for callers that may not allocate device memory.
//
// This entry point has no counterpart in CarlGergi/Layover; it is an addition of this library.
//
// Who needs it: a host program that owns the device's memory budget itself and therefore cannot
// let a library call cudaMalloc (or an allocating framework routine) on its behalf. Examples are
// a serving process that carved the whole device into its own arena at start-up, so that a later
// allocation would fail or fragment it; and a latency-critical loop that forbids allocator calls
// once it is warm, because cudaMalloc and cudaFree may synchronise the whole device. The regular
// entry point (`lb_attention_decode_bf16` in attention_mma.cu) takes its split-K scratch (partial
// outputs and per-(sequence, KV head) counters) from the caller, who has to allocate it; this one
// brings its own scratch: one file-scope `static __device__` array inside the library.
//
// Limits, which follow from that array's fixed size (LB_STATIC_SCRATCH_BYTES, 4 MiB + 16 KiB):
//   n_seqs * kv_heads                          <= LB_STATIC_MAX_COUNTERS (4096)
//   n_seqs * q_heads * splits * (dim + 2)      <= LB_STATIC_MAX_PARTIAL_FLOATS (1 Mi floats)
// A call beyond either limit is refused with LB_STATIC_ERR_TOO_LARGE and launches nothing.
//
// Things to know:
//   * Every GPU whose context loads this library holds the array until the process exits.
//   * The first call on each device, with that device current, looks up the array's address there
//     (cudaGetSymbolAddress) and raises the kernels' shared-memory limit on it; make that first call
//     outside any stream capture, and from one host thread at a time.
//   * All calls share the array and it keeps what the last call left. Each call clears the
//     counters it is about to use (a memset on the caller's stream), so a call that was torn
//     down half-way cannot poison the next. Two calls that overlap on the GPU (different streams
//     without ordering between them) race on the array: order them.
//   * It calls no cudaMalloc, cudaFree or allocating library routine, and neither does anything
//     it calls. Inputs and outputs are the caller's.
#pragma once
#include <cuda_runtime.h>

#define LB_STATIC_MAX_COUNTERS 4096
#define LB_STATIC_MAX_PARTIAL_FLOATS (1 << 20)
#define LB_STATIC_SCRATCH_BYTES (LB_STATIC_MAX_COUNTERS * 4 + LB_STATIC_MAX_PARTIAL_FLOATS * 4)

#define LB_STATIC_ERR_TOO_LARGE (-20)   // the batch needs more scratch than the static array holds
#define LB_STATIC_ERR_SETUP (-21)       // the array's device address could not be obtained
#define LB_STATIC_ERR_SHAPE (-22)       // head size, head counts or splits outside what the kernel takes

#ifdef __cplusplus
extern "C" {
#endif

// out[row, head, :] = attention of the single new token of each of `n_seqs` sequences over its
// paged keys and values (bfloat16, head size a multiple of 16 up to 256, at most 16 query heads per
// KV head). The arguments of `lb_attention_decode_bf16` without the scratch pointers and without
// `seq_list` (every sequence is served, in order). The result is that entry point's up to the order
// in which the splits are added: bit-identical wherever the regular entry merges through scratch
// memory too, and within rounding of it for head size 128 with 2, 4 or 8 splits, where the regular
// entry merges inside a thread-block cluster. A sequence whose ctx_len is 0 gets zeros.
// Returns 0, a cudaError_t (> 0) from the launch, or one of LB_STATIC_ERR_*.
int lb_attention_decode_bf16_static(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    const int* block_table, int table_width, const int* cu_q, const int* ctx_len,
                                    int n_seqs, int q_heads, int kv_heads, int dim, int page_tokens, float scale,
                                    int window, int splits, cudaStream_t stream);

// A sentence for each LB_STATIC_ERR_* code (a static string; never null).
const char* lb_attention_decode_static_strerror(int code);

#ifdef __cplusplus
}
#endif
