// Shared helpers of the sm_100a kernels: element types, rounding points, reductions.
//
// Every exported function is `extern "C"`, takes raw device pointers and a stream, launches
// asynchronously and returns the launch's cudaError_t as an int (0 = ok). Negative return
// values are refusals of a size or an alignment that the kernel does not support; the Python
// side turns both into exceptions, so that a wrong size never gives a wrong result.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LB_EXPORT extern "C" __attribute__((visibility("default")))

enum LbDtype { LB_F32 = 0, LB_BF16 = 1 };

// refusals (negative so that they cannot be mistaken for a cudaError_t)
#define LB_ERR_DTYPE (-1)
#define LB_ERR_SIZE (-2)
#define LB_ERR_ALIGN (-3)

typedef __nv_bfloat16 bf16;

// A request's record of fixed size on the device: int32 words, one row per state slot. Written
// whole when the request is admitted; the sampling kernel reads seed, counter and temperature,
// stores the token it chose and bumps the counter; the embedding kernel reads the last token of
// rows whose token the host has not seen yet.
#define LB_RECORD_WORDS 8
#define LB_RECORD_POSITION 0      // tokens the request holds once its newest sampled token is counted
#define LB_RECORD_SEED_LO 1
#define LB_RECORD_SEED_HI 2
#define LB_RECORD_COUNT 3         // tokens sampled so far
#define LB_RECORD_TEMPERATURE 4   // float bits; 0 = greedy
#define LB_RECORD_LAST_TOKEN 5

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  // value of `v` after a round trip through the storage type
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct Elem<bf16> {
  static __device__ __forceinline__ float load(const bf16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block in a fixed order (so that a row's result does not depend on the batch):
// butterfly inside each warp, then warp 0 adds the warps' partial sums in index order.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    scratch[32] = total;
  }
  __syncthreads();
  return scratch[32];
}

static inline int lb_last_error() { return (int)cudaGetLastError(); }

// Function attributes (the raised shared-memory limit of a kernel) belong to a device, not to the
// process: `first()` is true once per device, for the device that is current at the call.
struct LbPerDeviceOnce {
  static constexpr int MAX_DEVICES = 64;
  bool done[MAX_DEVICES] = {};
  int current() const {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return -1;
    return device;
  }
  bool first() {
    const int device = current();
    if (device < 0) return true;          // unknown device: configure again rather than not at all
    if (done[device]) return false;
    done[device] = true;
    return true;
  }
};

// ---- programmatic dependent launch
// Every kernel of this package is launched so that it may start while its predecessor in the
// stream is still running: its blocks set themselves up (and a matrix product already streams
// weights, which no kernel writes) and then wait in `pdl_wait()` until the predecessor has
// finished and its writes are visible. Every kernel calls `pdl_wait()` before it touches memory
// that an earlier kernel wrote or that a later kernel may still read, so completion is
// transitive along the stream. LAYOVER_B200_PDL=0 launches the plain way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
static inline bool lb_pdl_enabled() {
  static const bool enabled = [] {
    const char* v = std::getenv("LAYOVER_B200_PDL");
    return !(v && v[0] == '0');
  }();
  return enabled;
}

template <typename... KArgs, typename... Args>
static inline int lb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = lb_pdl_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// One lane's share of a head's sum of squares: eight elements of each half, as the per-head norm
// kernel and the fused projection epilogue both take it (the same expression, so the same bits).
__device__ __forceinline__ float lb_square_pair(float lo, float hi) { return lo * lo + hi * hi; }

// Thread-block clusters: blocks that hold parts of one result are launched as one cluster and hand
// their partial sums to one another through distributed shared memory.
// LAYOVER_B200_CLUSTER_REDUCE=0 sends split results through scratch memory and a counter instead.
static inline bool lb_cluster_reduce_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("LAYOVER_B200_CLUSTER_REDUCE");
    return !(v && v[0] == '0');
  }();
  return enabled;
}
__device__ __forceinline__ uint32_t lb_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t lb_map_to_rank(uint32_t smem_addr, uint32_t rank) {   // the same address in another block
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void lb_store_remote4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void lb_store_remote(uint32_t addr, float a) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ void lb_cluster_barrier() {    // every thread of every block of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// A launch with thread-block clusters of `cluster` blocks (every dimension divides the grid's).
template <typename... KArgs, typename... Args>
static inline int lb_launch_cluster_dims(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                         dim3 cluster, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = cluster.x;
  attribute[0].val.clusterDim.y = cluster.y;
  attribute[0].val.clusterDim.z = cluster.z;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = lb_pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// A launch with the blocks of one z column as a thread-block cluster of `cluster_z` blocks.
template <typename... KArgs, typename... Args>
static inline int lb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    unsigned cluster_z, Args... args) {
  return lb_launch_cluster_dims(kernel, grid, block, smem, stream, dim3(1, 1, cluster_z), args...);
}
