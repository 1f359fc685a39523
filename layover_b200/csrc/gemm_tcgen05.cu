// C[M, N] = A[M, K] * W[N, K]^T for bfloat16 operands on the 5th-generation tensor cores:
// TMA tiles (128-byte swizzle) -> shared memory -> tcgen05.mma with the accumulator in tensor
// memory -> tcgen05.ld -> registers -> global memory. 32-bit accumulation; C is bfloat16 or
// float32. The reference runs these products through cuBLAS (layover/model.py:110-113,148-150,182).
//
// One kernel, two orientations. Both operands are K-major, so either may sit on the 128-row
// side of the MMA:
//   many tokens (M > 128): tokens on the 128-row side, 256 (or 128) weight rows on the N side;
//   few tokens (decode):   128 weight rows on the 128-row side, the tokens (padded to 16..128) on
//                          the N side, so the tensor core's 128 rows are always full and the
//                          kernel is a pure stream of the weight matrix. When the weight has too
//                          few 128-row tiles to occupy the GPU, K is split over several blocks;
//                          each writes a 32-bit partial tile to scratch memory and the block that
//                          arrives last adds them in split order (a fixed order, so the result
//                          does not depend on timing) and resets the tile's counter.
//
// Block = 4 warps. Warp 0 lane 0 issues TMA loads through a ring of stages, warp 1 lane 0 issues
// the MMAs and frees stages with tcgen05.commit; all four warps run the epilogue (warp w owns
// tensor-memory lanes 32w..32w+31). Every wait on an mbarrier is bounded: when a limit runs out
// the block records an error code, lets copies in flight land, frees its tensor memory and
// returns; `lb_gemm_tcgen05_status` reports it.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;          // rows of the MMA's M side
constexpr int BK = 64;           // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 128;
constexpr int SMEM_BUDGET = 200 * 1024;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ int g_gemm_error = 0;   // 0 = ok; 1 producer, 2 mma, 3 epilogue wait ran out

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

// K-major operand tile with 128-byte swizzle, as TMA wrote it: rows of 128 bytes, groups of 8 rows
// 1024 bytes apart. Start address, leading offset (unused: 1), stride offset, version 1, layout 2.
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
  const uint32_t lo = ((smem_u32(tile) >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}
// bf16 x bf16 -> f32, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
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

// The few-token orientation keeps two blocks on an SM (half the shared memory each), so that a
// weight matrix with about as many tiles as SMs, or one split in two, still runs in one wave.
template <int BN, bool SWAP> struct Tile {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BUDGET = SWAP ? SMEM_BUDGET / 2 : SMEM_BUDGET;
  static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
  static constexpr int BLOCKS_PER_SM = SWAP ? 2 : 1;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// D[i, j] = sum_k Aop[i, k] Bop[j, k], i on the 128-row side. SWAP false: C[i, j] = D; true: C[j, i] = D.
template <int BN, bool SWAP, typename OutT>
__global__ void __launch_bounds__(THREADS, Tile<BN, SWAP>::BLOCKS_PER_SM)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OutT* __restrict__ C, long ldc, int rows_a, int rows_b, int K, int splits,
                    float* __restrict__ partials, unsigned* __restrict__ counters, bool vector_ok) {
  using T = Tile<BN, SWAP>;
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles_a = smem;
  uint8_t* tiles_b = smem + T::STAGES * T::A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + T::STAGES * T::STAGE_BYTES);
  uint64_t* empty = full + T::STAGES;
  uint64_t* tmem_full = empty + T::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  uint32_t* flag = tmem_slot + 1;   // [0] failed, [1] this block is the last of its tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN, split = blockIdx.z;
  const int total_kb = (K + BK - 1) / BK;
  const int kb_begin = (int)((long)total_kb * split / splits), kb_end = (int)((long)total_kb * (split + 1) / splits);
  const int n_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(tmem_full, 1);
    flag[0] = 0; flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, T::TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  if (warp == 0 && lane == 0) {
    // ---------------- producer. The weights are written by no kernel, so the first ring of weight
    // tiles is requested before waiting for the kernel that produces the activations.
    const int early = n_kb < T::STAGES ? n_kb : T::STAGES;
    for (int i = 0; i < early; ++i) {
      mbar_expect_tx(&full[i], T::STAGE_BYTES);
      if (SWAP) tma_load_2d(tiles_a + i * T::A_BYTES, &map_a, &full[i], (kb_begin + i) * BK, m0);
      else tma_load_2d(tiles_b + i * T::B_BYTES, &map_b, &full[i], (kb_begin + i) * BK, n0);
    }
    pdl_wait();
    for (int i = 0; i < early; ++i) {
      if (SWAP) tma_load_2d(tiles_b + i * T::B_BYTES, &map_b, &full[i], (kb_begin + i) * BK, n0);
      else tma_load_2d(tiles_a + i * T::A_BYTES, &map_a, &full[i], (kb_begin + i) * BK, m0);
    }
    for (int i = early; i < n_kb; ++i) {
      const int s = i % T::STAGES;
      const uint32_t phase = (i / T::STAGES) & 1;
      if (!mbar_wait(&empty[s], phase ^ 1)) { atomicCAS(&g_gemm_error, 0, 1); flag[0] = 1; break; }
      mbar_expect_tx(&full[s], T::STAGE_BYTES);
      tma_load_2d(tiles_a + s * T::A_BYTES, &map_a, &full[s], (kb_begin + i) * BK, m0);
      tma_load_2d(tiles_b + s * T::B_BYTES, &map_b, &full[s], (kb_begin + i) * BK, n0);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    constexpr uint32_t idesc = instr_desc(BN);
    bool ok = true;
    for (int i = 0; i < n_kb && ok; ++i) {
      const int s = i % T::STAGES;
      const uint32_t phase = (i / T::STAGES) & 1;
      if (!mbar_wait(&full[s], phase)) { atomicCAS(&g_gemm_error, 0, 2); flag[0] = 1; ok = false; break; }
      fence_after_sync();
      const uint64_t a_desc = smem_desc(tiles_a + s * T::A_BYTES), b_desc = smem_desc(tiles_b + s * T::B_BYTES);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)
        umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);  // +32 bytes per K step
      umma_commit(&empty[s]);
    }
    if (ok) umma_commit(tmem_full);
  }
  __syncwarp();
  pdl_wait();   // the epilogue writes memory that earlier kernels may still be reading

  // ---------------- epilogue: every warp reads its 32 lanes of the accumulator
  const bool ready = mbar_wait(tmem_full, 0);
  if (!ready) { atomicCAS(&g_gemm_error, 0, 3); flag[0] = 1; }
  fence_after_sync();
  const int row = warp * 32 + lane;                       // row of the 128-row side
  const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
  const int valid_cols = min(BN, rows_b - n0);
  const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
  float* my_partial = partials ? partials + ((size_t)tile_id * splits + split) * BN * BM : nullptr;

  if (ready) {
    for (int c = 0; c < BN; c += 16) {
      if (c >= valid_cols) break;                           // uniform over the block
      float v[16];
      tmem_ld16(lane_base + c, v);
      if (splits > 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (c + i < valid_cols) my_partial[(size_t)(c + i) * BM + row] = v[i];
      } else if (SWAP) {
        if (m0 + row < rows_a) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c + i < valid_cols) store_one<OutT>(C + (size_t)(n0 + c + i) * ldc + m0 + row, v[i]);
        }
      } else {
        if (m0 + row < rows_a) {
          OutT* dst = C + (size_t)(m0 + row) * ldc + n0 + c;
          if (vector_ok && c + 16 <= valid_cols) {
            store_row16<OutT>(dst, v);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (c + i < valid_cols) store_one<OutT>(dst + i, v[i]);
          }
        }
      }
    }
  }

  if (splits > 1) {
    // the block that arrives last at this tile's counter adds the partial tiles in split order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned arrived = atomicAdd(&counters[tile_id], 1u);
      flag[1] = (arrived == (unsigned)splits - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (flag[1]) {
      __threadfence();
      const float* tile_partials = partials + (size_t)tile_id * splits * BN * BM;
      if (m0 + row < rows_a) {
        // eight columns and four splits at a time: those 32 loads do not depend on one another,
        // and every element is still summed in split order
        for (int j0 = 0; j0 < valid_cols; j0 += 8) {
          float sum[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) sum[u] = 0.f;
          for (int s0 = 0; s0 < splits; s0 += 4) {
            float part[4][8];
#pragma unroll
            for (int ds = 0; ds < 4; ++ds) {
              const float* src = tile_partials + ((size_t)(s0 + ds) * BN + j0) * BM + row;
#pragma unroll
              for (int u = 0; u < 8; ++u)
                part[ds][u] = (s0 + ds < splits && j0 + u < valid_cols) ? src[(size_t)u * BM] : 0.f;
            }
#pragma unroll
            for (int ds = 0; ds < 4; ++ds)
#pragma unroll
              for (int u = 0; u < 8; ++u) sum[u] += part[ds][u];
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (j0 + u < valid_cols) {
              if (SWAP) store_one<OutT>(C + (size_t)(n0 + j0 + u) * ldc + m0 + row, sum[u]);
              else store_one<OutT>(C + (size_t)(m0 + row) * ldc + n0 + j0 + u, sum[u]);
            }
          }
        }
      }
      if (threadIdx.x == 0) counters[tile_id] = 0;   // ready for the next launch
    }
  }

  // ---------------- teardown
  fence_before_sync();
  __syncthreads();
  if (flag[0]) {
    // a wait ran out: give copies still in flight time to land before the block's memory goes away
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

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

// rows x K bf16 matrix with row stride `ld` elements; box = 64 (K) x box_rows, 128-byte swizzle, zero fill
bool make_map(CUtensorMap* map, const void* base, long rows, long K, long ld, int box_rows) {
  auto encode = encode_fn();
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool SWAP, typename OutT>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, void* C, long ldc, int rows_a, int rows_b, int K,
           int splits, float* partials, unsigned* counters, bool vector_ok, cudaStream_t stream) {
  using T = Tile<BN, SWAP>;
  auto kernel = gemm_tcgen05_kernel<BN, SWAP, OutT>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM) != cudaSuccess)
      return lb_last_error();
    configured = true;
  }
  dim3 grid((rows_a + BM - 1) / BM, (rows_b + BN - 1) / BN, splits);
  const int code = lb_launch(kernel, grid, dim3(THREADS), (size_t)T::SMEM, stream, map_a, map_b, (OutT*)C, ldc, rows_a,
                             rows_b, K, splits, partials, counters, vector_ok);
  return code ? code : lb_last_error();
}

template <bool SWAP, typename OutT>
int launch_bn(int bn, const CUtensorMap& a, const CUtensorMap& b, void* C, long ldc, int rows_a, int rows_b, int K,
              int splits, float* partials, unsigned* counters, bool vector_ok, cudaStream_t stream) {
  switch (bn) {
    case 16: return launch<16, SWAP, OutT>(a, b, C, ldc, rows_a, rows_b, K, splits, partials, counters, vector_ok, stream);
    case 32: return launch<32, SWAP, OutT>(a, b, C, ldc, rows_a, rows_b, K, splits, partials, counters, vector_ok, stream);
    case 64: return launch<64, SWAP, OutT>(a, b, C, ldc, rows_a, rows_b, K, splits, partials, counters, vector_ok, stream);
    case 128: return launch<128, SWAP, OutT>(a, b, C, ldc, rows_a, rows_b, K, splits, partials, counters, vector_ok, stream);
    case 256: return launch<256, SWAP, OutT>(a, b, C, ldc, rows_a, rows_b, K, splits, partials, counters, vector_ok, stream);
  }
  return LB_ERR_SIZE;
}
}  // namespace

// The error code a kernel recorded when one of its bounded waits ran out (0 = none); clears it.
LB_EXPORT int lb_gemm_tcgen05_status() {
  int code = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&code, g_gemm_error, sizeof(int)) != cudaSuccess) return -100;
  if (code) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  return code;
}

// Whether this product can run here: addresses 16-byte aligned, row strides multiples of 8 elements.
LB_EXPORT int lb_gemm_tcgen05_supports(const void* A, const void* W, int K, long lda, long ldw) {
  return ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0) && lda % 8 == 0 && ldw % 8 == 0 && K >= 1 && lda >= K &&
         ldw >= K;
}

// C[M, N] = A[M, K] W[N, K]^T. out_dtype: LB_BF16 or LB_F32. `scratch` (floats) and `counters`
// (zeroed once by the caller, `n_counters` of them) serve the split-K path; without them K is
// never split. `sm_count` sizes the split; `max_splits` > 0 caps it.
LB_EXPORT int lb_gemm_tcgen05(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K, long lda,
                              long ldw, long ldc, float* scratch, long scratch_floats, unsigned* counters,
                              int n_counters, int sm_count, int max_splits, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!lb_gemm_tcgen05_supports(A, W, K, lda, ldw)) return LB_ERR_ALIGN;
  if (out_dtype != LB_BF16 && out_dtype != LB_F32) return LB_ERR_DTYPE;
  const bool swap = M <= 128;
  CUtensorMap map_a, map_b;
  int bn, rows_a, rows_b, splits = 1;
  if (swap) {
    bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    rows_a = N; rows_b = M;
    if (!make_map(&map_a, W, N, K, ldw, BM) || !make_map(&map_b, A, M, K, lda, bn)) return LB_ERR_ALIGN;
    const int tiles = (N + BM - 1) / BM;
    const int total_kb = (K + BK - 1) / BK;
    if (scratch && counters && tiles <= n_counters && tiles < sm_count) {
      // One block per SM streams a weight matrix at close to full bandwidth, and every further
      // split adds a partial tile to write, a fence, a counter and a longer sum, which at these
      // sizes cost more than the extra blocks win (measured on 2560..9728-wide weights: 8 splits
      // of a 20-tile matrix beat 15; a 152-tile matrix is fastest unsplit). Wider token tiles
      // make the partial tiles bigger, so they split less.
      const int cap = bn <= 16 ? 8 : (bn <= 32 ? 4 : 2);
      splits = (sm_count + tiles - 1) / tiles;
      if (splits > cap) splits = cap;
      if (splits > total_kb / 4) splits = total_kb / 4;         // at least four K blocks per split
      if (max_splits > 0 && splits > max_splits) splits = max_splits;
      const long per_split = (long)tiles * bn * BM;
      if (splits > 1 && per_split * splits > scratch_floats) splits = (int)(scratch_floats / per_split);
      if (splits < 1) splits = 1;
    }
  } else {
    // 256-wide tiles: half the shared-memory traffic per flop of 128-wide ones, which measured
    // slower at every size even with two blocks per SM
    bn = N > 128 ? 256 : 128;
    rows_a = M; rows_b = N;
    if (!make_map(&map_a, A, M, K, lda, BM) || !make_map(&map_b, W, N, K, ldw, bn)) return LB_ERR_ALIGN;
  }
  float* partials = splits > 1 ? scratch : nullptr;
  const int elem = out_dtype == LB_BF16 ? 2 : 4;
  const bool vector_ok = ((uintptr_t)C % 16 == 0) && ((ldc * elem) % 16 == 0);
  if (swap) {
    if (out_dtype == LB_BF16)
      return launch_bn<true, bf16>(bn, map_a, map_b, C, ldc, rows_a, rows_b, K, splits, partials, counters, vector_ok, stream);
    return launch_bn<true, float>(bn, map_a, map_b, C, ldc, rows_a, rows_b, K, splits, partials, counters, vector_ok, stream);
  }
  if (out_dtype == LB_BF16)
    return launch_bn<false, bf16>(bn, map_a, map_b, C, ldc, rows_a, rows_b, K, 1, nullptr, nullptr, vector_ok, stream);
  return launch_bn<false, float>(bn, map_a, map_b, C, ldc, rows_a, rows_b, K, 1, nullptr, nullptr, vector_ok, stream);
}
