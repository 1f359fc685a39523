// What the kernels that drive the 5th-generation tensor cores share: PTX wrappers for mbarriers,
// TMA tile loads, tensor memory and tcgen05.mma, the shared-memory and instruction descriptors of
// K-major bfloat16 operands with the 128-byte swizzle, the roundings of the reference's bfloat16
// tensors, and the host-side tensor-map encoder. Every wait is bounded: `mbar_wait` returns false
// when its limit runs out and the caller records that, lets copies in flight land, frees its tensor
// memory and leaves.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include <functional>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int BM = 128;          // rows of the MMA's M side
constexpr int BK = 64;           // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// true when the phase with the given parity has completed; false when the limit ran out
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin > 1024) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier once every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- two blocks of a cluster as one MMA unit (cta_group::2). The even block of the pair (the
// leader) issues the MMAs; each block stages its own 128 rows of either operand at the same
// shared-memory offsets, and each gets the accumulator rows of its own 128 rows of the M side.
// A copy into this block's shared memory that reports its bytes to a barrier of either block of the
// pair (`bar_cluster` is a shared::cluster address, as `mapa` gives it).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
// one warp of each block of the pair, the same warp in both
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  const uint32_t zero = 0;       // no output lane is switched off
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero)
      : "memory");
}
// arrives on the barrier at this offset in every block of `block_mask` (bit r: the cluster's block r)
// once every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t block_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(block_mask) : "memory");
}
// an arrival on a barrier of any block of the cluster (`bar_cluster` from `mapa`)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

// two loads of 16 columns each under one wait
__device__ __forceinline__ void tmem_ld16_two(uint32_t taddr_a, uint32_t taddr_b, float (&a)[16], float (&b)[16]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%32];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%33];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr_a), "r"(taddr_b)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) { a[i] = __uint_as_float(r[i]); b[i] = __uint_as_float(r[16 + i]); }
}

// K-major operand tile with 128-byte swizzle, as TMA wrote it: rows of 128 bytes, groups of 8 rows
// 1024 bytes apart. Start address, leading offset (unused: 1), stride offset, version 1, layout 2.
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
  const uint32_t lo = ((smem_u32(tile) >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}
// bf16 x bf16 -> f32, both K-major, M = m (128; 256 for a pair of blocks), N = n
__host__ __device__ constexpr uint32_t instr_desc(int n, int m = BM) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <typename OutT> __device__ __forceinline__ void store_one(OutT* p, float v);
template <> __device__ __forceinline__ void store_one<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_one<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename OutT> __device__ __forceinline__ void store_row16(OutT* p, const float (&v)[16]);
template <> __device__ __forceinline__ void store_row16<float>(float* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}
template <> __device__ __forceinline__ void store_row16<bf16>(bf16* p, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&pair);
  }
  reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// silu(g) * u as the reference's bfloat16 tensors compute it: the two projections round to bf16,
// the activation rounds to bf16, the product rounds when it is stored (layover/model.py:152-153).
__device__ __forceinline__ float swiglu_bf16(float g, float u) {
  g = __bfloat162float(__float2bfloat16_rn(g));
  u = __bfloat162float(__float2bfloat16_rn(u));
  const float act = __bfloat162float(__float2bfloat16_rn(g / (1.0f + expf(-g))));
  return act * u;
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// What the epilogue for fused q/k/v projections needs: a 128-row tile is one head of 128 dims
// there, and whoever owns a token norms, rotates and stores the head's row of it.
struct HeadsEpilogue {
  const float* q_norm_w;      // [128]
  const float* k_norm_w;
  const float* rope_table;    // [tokens][2][64]: cos, sin
  const int* slot_map;        // [tokens]: page * page_tokens + slot
  bf16* q_out;                // [tokens][q_heads][128]
  bf16* k_pool;               // [pages][kv_heads][page_tokens][128]
  bf16* v_pool;
  int q_heads, kv_heads, page_tokens;
  float eps;
};

// ------------------------------------------------------------------ host side
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (PFN_cuTensorMapEncodeTiled_v12000)p;
  }();
  return fn;
}

// rows x K bf16 matrix with row stride `ld` elements; box = 64 (K) x box_rows, 128-byte swizzle, zero fill.
// Encoded maps are kept by (address, shape, stride, box): a weight's map is made once per process, and
// an activation buffer that comes back at the same address (a captured step's, an allocator's reuse)
// finds its map again. The table is small and guarded by one lock.
struct MapKey {
  const void* base;
  long rows, K, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    h = h * 1000003u ^ std::hash<long>()(k.rows);
    h = h * 1000003u ^ std::hash<long>()(k.K);
    h = h * 1000003u ^ std::hash<long>()(k.ld);
    return h * 1000003u ^ std::hash<int>()(k.box_rows);
  }
};

bool make_map(CUtensorMap* map, const void* base, long rows, long K, long ld, int box_rows) {
  static std::mutex lock;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> known;
  const MapKey key{base, rows, K, ld, box_rows};
  {
    std::lock_guard<std::mutex> guard(lock);
    auto found = known.find(key);
    if (found != known.end()) { *map = found->second; return true; }
  }
  auto encode = encode_fn();
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  std::lock_guard<std::mutex> guard(lock);
  if (known.size() > 4096) known.clear();      // far more than a model's weights: start over rather than grow for ever
  known.emplace(key, *map);
  return true;
}
}  // namespace
