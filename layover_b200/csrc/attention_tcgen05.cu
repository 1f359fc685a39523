// Paged grouped-query attention for prompt portions in bfloat16 on the 5th-generation tensor cores:
// both products of attention (S = Q K^T and O = P V) are tcgen05.mma with accumulators in tensor
// memory, K and V pages come by TMA straight from the block table, and the softmax runs one thread
// per query row. The reference gathers the history out of its pool and calls a library kernel for
// prompts (layover/model.py:84-90).
//
// Two kernels over tiles of 128 consecutive tokens of a sequence:
//   attention_tcgen05_pair_kernel  two query heads that share a KV head per block (an even number
//                                  of query heads per KV head), probabilities kept in tensor memory
//   attention_tcgen05_kernel       one query head per block, probabilities through shared memory
//
// Common to both: warp 0 walks the block table and issues one 5-D TMA copy per page and half of the
// head, one copy per lane (the whole cache group's pool is ONE tensor map: dim, slot, KV head, page,
// layer x {K, V}); warp 1 lane 0 issues the MMAs; the softmax warps own one query row per thread:
// they read the row's 128 scores from tensor memory, keep the running maximum and sum, write the
// probabilities as the bf16 A operand of the second product and rescale the output only when the
// maximum has grown by more than 2^8 (the accumulated values stay exact relative to a reference
// maximum; the final division uses the same reference). Every mbarrier wait is bounded.
//
// Limits: head size 128, page size a multiple of 8 that divides 128; anything else is refused (the
// mma.sync kernels of attention_mma.cu take it). Decode steps use attention_mma.cu's split kernel:
// two tcgen05 formulations of it (heads on the MMA rows, keys on the MMA rows) were measured at
// 40 us against 28 us at batch 8 and 3.1 against 5.1 TB/s at batch 64 and are not kept.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int ROWS = 128;        // query rows per block (the MMA's M)
constexpr int KEYS = 128;        // keys per tile (N of the first product, K of the second)
constexpr int DIM = 128;         // head size
constexpr int HALF_BYTES = ROWS * 128;          // one 64-column half of a 128-row operand: 16 KiB
constexpr int TILE_BYTES = 2 * HALF_BYTES;      // 32 KiB
constexpr int KV_STAGES = 2;
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 20;
constexpr float RESCALE_THRESHOLD = 8.0f;       // in log2 units

__device__ int g_attn_error = 0;   // 0 = ok; which wait ran out otherwise

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if (spin > 1024) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {   // one look, never suspends
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 64 columns of this thread's lane, no wait: tmem_wait_ld() must come before the values are used.
__device__ __forceinline__ void tmem_ld64_nowait(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16_nowait(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (bf16, two elements of K per 32-bit column) is read from tensor memory
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The maximum of a row's scores over four chains that do not wait for one another (one chain of 128
// dependent comparisons costs more than the exponentials that follow).
template <int N>
__device__ __forceinline__ float row_max(const float (&s)[N]) {
  float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int e = 0; e < N; e += 4) {
#pragma unroll
    for (int k = 0; k < 4; ++k) m[k] = fmaxf(m[k], s[e + k]);
  }
  return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared-memory matrix descriptors, 128-byte swizzle, version 1.
// K-major (rows of 128 bytes, 8-row groups 1024 bytes apart): Q, K and P.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}
// MN-major (the same bytes read with the 128-byte rows running along N): V as the B operand of
// O = P V. Leading offset: from one 64-column block of the head to the next (the other half of the
// tile); stride offset: from one group of 8 keys to the next.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  const uint32_t lo = ((addr >> 4) & 0x3FFFu) | ((uint32_t)(HALF_BYTES >> 4) << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}
// bf16 x bf16 -> f32, M = 128, N = 128; b_mn: B is MN-major
constexpr uint32_t instr_desc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

constexpr int TABLE_CACHE = 1024;   // block-table entries the producer warp keeps in shared memory

// The producer warp copies the pages of its tiles from the block table to shared memory first: a
// page id read from global memory in front of every TMA copy would put a round trip to the L2 into
// the issue loop, sixteen times per tile. Entries past the cache (or past the table, which are
// masked anyway) fall back to a clamped global read.
__device__ __forceinline__ void cache_pages(int* cached, const int* __restrict__ table, int table_width, int first_page,
                                            int n_pages, int lane) {
  for (int i = lane; i < min(n_pages, TABLE_CACHE); i += 32) cached[i] = table[min(first_page + i, table_width - 1)];
  __syncwarp();
}
__device__ __forceinline__ int page_at(const int* cached, const int* __restrict__ table, int table_width, int first_page,
                                       int index) {
  const int local = index - first_page;
  return local < TABLE_CACHE ? cached[local] : table[min(index, table_width - 1)];
}

struct Args {
  bf16* out;
  const int* block_table;
  int table_width;
  const int* cu_q;
  const int* ctx_len;
  const int* tile_seq;      // the tiles of 128 queries: sequence and first query of each
  const int* tile_q0;
  int q_heads, kv_heads, page_tokens, window;
  int layer2;               // 2 * layer: the K plane of this layer in the pool's last dimension
  float scale_log2;
};

// The producer warp's loop. K and V tiles are requested independently, each as soon as its own
// stage is free: taken in turn, the K tile of a later step would queue behind a V stage that the
// second product frees late. A tile is 128 / page_tokens pages x 2 halves of the head = up to 32
// TMA copies; one thread issuing them one after the other spends over a hundred cycles on each,
// more than the tile's arithmetic takes, so every lane issues one copy of the tile in the same
// instruction. Lane 0 watches the barriers. `code` marks the kernel in the error word if the wait
// runs out.
template <int STAGES>
__device__ __forceinline__ void produce_kv(const CUtensorMap* kv_map, const Args& args, uint8_t* k_s, uint8_t* v_s,
                                           uint64_t* k_full, uint64_t* k_empty, uint64_t* v_full, uint64_t* v_empty,
                                           const int* page_cache, const int* table, int tile_begin, int n_tiles,
                                           int kv_head, volatile uint32_t* flag, int code, int lane) {
  const int pages_per_tile = KEYS / args.page_tokens;
  const int pg = lane >> 1, half = lane & 1;             // this lane's copy within a tile
  const bool mine = pg < pages_per_tile;
  int next_k = 0, next_v = 0;
  uint32_t idle = 0;
  while (next_k < n_tiles || next_v < n_tiles) {
    bool moved = false;
#pragma unroll
    for (int kind = 0; kind < 2; ++kind) {
      const int i = kind ? next_v : next_k;
      if (i >= n_tiles) continue;
      const int stage = i % STAGES;
      uint64_t* empty = kind ? &v_empty[stage] : &k_empty[stage];
      uint64_t* full = kind ? &v_full[stage] : &k_full[stage];
      int ready = 0;
      if (lane == 0) {
        ready = mbar_test(empty, ((i / STAGES) & 1) ^ 1) ? 1 : 0;
        if (ready) mbar_expect_tx(full, TILE_BYTES);
      }
      ready = __shfl_sync(0xffffffffu, ready, 0);
      if (!ready) continue;
      if (mine) {
        uint8_t* dst = (kind ? v_s : k_s) + stage * TILE_BYTES;
        const int page = page_at(page_cache, table, args.table_width, tile_begin * pages_per_tile,
                                 (tile_begin + i) * pages_per_tile + pg);
        tma_load_5d(dst + half * HALF_BYTES + pg * args.page_tokens * 128, kv_map, full, half * 64, 0, kv_head, page,
                    args.layer2 + kind);
      }
      if (kind) ++next_v; else ++next_k;
      moved = true;
    }
    int stop = 0;
    if (lane == 0) {
      if (moved) {
        idle = 0;
      } else if (++idle > SPIN_LIMIT) {
        atomicCAS(&g_attn_error, 0, code); flag[0] = 1;
      } else {
        __nanosleep(idle > 4096 ? 256 : 20);    // leave the issue slots to the softmax warps of this scheduler
      }
      stop = flag[0] ? 1 : 0;
    }
    if (__shfl_sync(0xffffffffu, stop, 0)) break;
  }
}

constexpr int SMEM_BYTES = TILE_BYTES * (2 + 2 * KV_STAGES) + 1024 + 512 + TABLE_CACHE * 4;   // Q, P, K and V stages, slack, barriers, table

__global__ void __launch_bounds__(THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                         const Args args) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;
  uint8_t* p_s = q_s + TILE_BYTES;
  uint8_t* k_s = p_s + TILE_BYTES;                       // [KV_STAGES][TILE_BYTES]
  uint8_t* v_s = k_s + KV_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + KV_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2] scores of a tile are in tensor memory
  uint64_t* s_empty = bars + 11;      // [2] the softmax has read them
  uint64_t* p_full = bars + 13;       // the probabilities are in shared memory, the output is rescaled
  uint64_t* pv_done = bars + 14;      // the second product of a tile is finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* flag = tmem_slot + 1;   // [0] a wait ran out, [1] last block of its (sequence, KV head)
  int* page_cache = reinterpret_cast<int*>(bars) + 128;   // after the 512 bytes of barriers

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- what this block works on
  // heads run fastest and the tile list is walked backwards: within a sequence later tiles have
  // more keys to visit, and the longest jobs should start first
  const int group = args.q_heads / args.kv_heads;
  const int tile_index = gridDim.y - 1 - blockIdx.y;
  const int seq = args.tile_seq[tile_index], q0 = args.tile_q0[tile_index];
  const int head = blockIdx.x, kv_head = head / group;
  const int row0 = args.cu_q[seq], q_len = args.cu_q[seq + 1] - row0, ctx = args.ctx_len[seq];
  const int n_rows = min(ROWS, q_len - q0);
  const int p_first = ctx - q_len + q0, p_last = p_first + n_rows - 1;
  const int key_lo = args.window > 0 ? max(0, p_first - args.window + 1) : 0;
  const int tile_begin = key_lo / KEYS, tile_end = p_last / KEYS + 1;
  const int q_row = row0 + q0;                             // row of q viewed as [tokens, heads * dim]
  const int n_tiles_mine = max(0, tile_end - tile_begin);
  const int* table = args.block_table + (size_t)seq * args.table_width;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    flag[0] = 0; flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;            // two score buffers of 128 columns
  const uint32_t tmem_o = tmem_base + 256;      // the output accumulator, 128 columns
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    const int pages_per_tile = KEYS / args.page_tokens;
    if (n_tiles_mine > 0) cache_pages(page_cache, table, args.table_width, tile_begin * pages_per_tile, n_tiles_mine * pages_per_tile, lane);
    if (n_tiles_mine > 0) {
      // ---------------- producer: the query tile, then K and V page by page
      if (lane == 0) {
        mbar_expect_tx(q_full, TILE_BYTES);
        for (int half = 0; half < 2; ++half)
          tma_load_2d(q_s + half * HALF_BYTES, &q_map, q_full, head * DIM + half * 64, q_row);
      }
      produce_kv<KV_STAGES>(&kv_map, args, k_s, v_s, k_full, k_empty, v_full, v_empty, page_cache, table, tile_begin,
                            n_tiles_mine, kv_head, flag, 1, lane);
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles_mine > 0) {
      // ---------------- MMA issuer: S(i + 1) = Q K^T is issued before O += P(i) V, so that the
      // softmax of one tile overlaps the first product of the next
      constexpr uint32_t idesc_s = instr_desc(false), idesc_o = instr_desc(true);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) { atomicCAS(&g_attn_error, 0, 2); flag[0] = 1; }
      auto issue_s = [&](int i) {
        const int stage = i % KV_STAGES, buf = i & 1;
        if (!mbar_wait(&k_full[stage], (i / KV_STAGES) & 1) || !mbar_wait(&s_empty[buf], ((i >> 1) & 1) ^ 1)) {
          atomicCAS(&g_attn_error, 0, 3); flag[0] = 1; return false;
        }
        fence_after_sync();
        const uint32_t q_addr = smem_u32(q_s), k_addr = smem_u32(k_s + stage * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < DIM / 16; ++ks) {
          const uint32_t off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          umma_bf16(tmem_s + buf * 128, desc_k_major(q_addr + off), desc_k_major(k_addr + off), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[buf]);
        umma_commit(&k_empty[stage]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int i = 0; i < n_tiles_mine && ok; ++i) {
        if (i + 1 < n_tiles_mine) ok = issue_s(i + 1);
        if (!ok) break;
        const int stage = i % KV_STAGES;
        if (!mbar_wait(p_full, i & 1) || !mbar_wait(&v_full[stage], (i / KV_STAGES) & 1)) {
          atomicCAS(&g_attn_error, 0, 4); flag[0] = 1; break;
        }
        fence_after_sync();
        const uint32_t p_addr = smem_u32(p_s), v_addr = smem_u32(v_s + stage * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < KEYS / 16; ++ks) {
          const uint32_t a_off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;     // 16 keys along P's rows
          const uint32_t b_off = ks * 16 * 128;                               // 16 key rows of V
          umma_bf16(tmem_o, desc_k_major(p_addr + a_off), desc_mn_major(v_addr + b_off), idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(pv_done);
        umma_commit(&v_empty[stage]);
      }
    }
  } else {
    // ---------------- softmax and epilogue: one query row per thread
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int p_row = p_first + row;                          // rows past n_rows are ballast
    const float c = args.scale_log2;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int i = 0; i < n_tiles_mine && ok; ++i) {
      const int tile = tile_begin + i, buf = i & 1, stage = i % KV_STAGES;
      const int key0 = tile * KEYS;
      if (!mbar_wait(&s_full[buf], (i >> 1) & 1)) { atomicCAS(&g_attn_error, 0, 5); flag[0] = 1; ok = false; break; }
      fence_after_sync();
      // the tile needs the comparisons if it reaches past the block's first position, starts before
      // the first visible key, or a window cuts it
      const bool masked = key0 + KEYS - 1 > p_first || key0 < key_lo || args.window > 0;
      float s[KEYS];
#pragma unroll
      for (int ch = 0; ch < KEYS / 16; ++ch) {
        float v[16];
        tmem_ld16(tmem_s + buf * 128 + lane_addr + ch * 16, v);
#pragma unroll
        for (int e = 0; e < 16; ++e) s[ch * 16 + e] = v[e];
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[buf]);
      float tile_max = -INFINITY;
      if (masked) {
#pragma unroll
        for (int e = 0; e < KEYS; ++e) {
          const int key = key0 + e;
          const bool seen = key <= p_row && key >= key_lo && (args.window <= 0 || p_row - key < args.window);
          if (!seen) s[e] = -INFINITY;
        }
      }
      tile_max = row_max(s);
      // The reference maximum only moves when the true one has outgrown it by 2^8: the accumulated
      // output then needs no rescaling for most tiles. A warp rescales together (tensor-memory
      // loads and stores are warp-wide), every lane by its own factor.
      const bool grow = (tile_max - m_ref) * c > RESCALE_THRESHOLD || (m_ref == -INFINITY && tile_max > -INFINITY);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      // The exponentials need only the reference maximum, so they are taken before waiting for the
      // previous tile's second product; that product must be done before the probabilities in
      // shared memory are overwritten or the output is touched.
      const float m_new = grow ? tile_max : m_ref;
      const float factor = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_new) * c);
      const float neg_base = (m_new == -INFINITY) ? 0.f : -m_new * c;
      uint32_t w[KEYS / 2];
      float part_sum[4] = {0.f, 0.f, 0.f, 0.f};           // four chains of additions side by side
#pragma unroll
      for (int e = 0; e < KEYS / 2; ++e) {
        const float a = fast_exp2(fmaf(s[2 * e], c, neg_base));
        const float b = fast_exp2(fmaf(s[2 * e + 1], c, neg_base));
        part_sum[e & 3] += a + b;
        const __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
        w[e] = *reinterpret_cast<const uint32_t*>(&pair);
      }
      const float tile_sum = (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
      l_sum = l_sum * factor + tile_sum;
      m_ref = m_new;
      if (i > 0 && !mbar_wait(pv_done, (i - 1) & 1)) { atomicCAS(&g_attn_error, 0, 6); flag[0] = 1; ok = false; break; }
      fence_after_sync();
      if (any_grow && i > 0) {
#pragma unroll
        for (int ch = 0; ch < DIM / 16; ++ch) {
          float v[16];
          tmem_ld16(tmem_o + lane_addr + ch * 16, v);
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] *= factor;
          tmem_st16(tmem_o + lane_addr + ch * 16, v);
        }
      }
      // probabilities as bf16 into the A operand of the second product: row `row`, 16-byte pieces
      // of 8 keys, swizzled like every 128-byte row
#pragma unroll
      for (int piece = 0; piece < KEYS / 8; ++piece) {
        const int half = piece >> 3, chunk = piece & 7;
        uint8_t* dst = p_s + half * HALF_BYTES + row * 128 + ((chunk ^ (row & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = make_uint4(w[4 * piece], w[4 * piece + 1], w[4 * piece + 2], w[4 * piece + 3]);
      }
      // V rows of keys that are not part of the context may hold anything (a stale or poisoned
      // page): zero them, since 0 x NaN would still be NaN. Only boundary tiles have such rows.
      const int limit = p_last + 1;
      if (key0 + KEYS > limit || key0 < key_lo) {
        if (!mbar_wait(&v_full[stage], (i / KV_STAGES) & 1)) { atomicCAS(&g_attn_error, 0, 7); flag[0] = 1; ok = false; break; }
        const int key = key0 + row;
        if (key >= limit || key < key_lo) {
          uint8_t* vrow = v_s + stage * TILE_BYTES + row * 128;
#pragma unroll
          for (int chunk = 0; chunk < 8; ++chunk) {
            *reinterpret_cast<uint4*>(vrow + chunk * 16) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vrow + HALF_BYTES + chunk * 16) = make_uint4(0, 0, 0, 0);
          }
        }
      }
      fence_async_smem();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }

    // ---- the block's result: wait for the last second product, read the row, divide, store
    if (ok && n_tiles_mine > 0) {
      if (!mbar_wait(pv_done, (n_tiles_mine - 1) & 1)) { atomicCAS(&g_attn_error, 0, 8); flag[0] = 1; ok = false; }
      fence_after_sync();
    }
    if (ok) {
      // tensor-memory loads are warp-wide: every lane reads its row, rows of the tile only are stored
      const bool valid = row < n_rows;
      bf16* dst = args.out + ((size_t)(q_row + (valid ? row : 0)) * args.q_heads + head) * DIM;
      const float inv = 1.0f / l_sum;
#pragma unroll
      for (int ch = 0; ch < DIM / 16; ++ch) {
        float v[16];
        if (n_tiles_mine > 0) {
          tmem_ld16(tmem_o + lane_addr + ch * 16, v);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0.f;
        }
        if (!valid) continue;
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * e] * inv, v[2 * e + 1] * inv);
          w[e] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        reinterpret_cast<uint4*>(dst + ch * 16)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(dst + ch * 16)[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }

  // ---------------- teardown
  fence_before_sync();
  __syncthreads();
  if (flag[0]) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies in flight land
    __syncthreads();
  }
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------- prompt portions, two heads per block
// The kernel for prompt portions where an even number of query heads shares a KV head. A block
// takes the same 128 tokens of TWO such heads: each head has its own query tile, score and output
// accumulators in tensor memory and its own softmax warpgroup, and both read the same K and V
// tiles. The MMA thread alternates between the heads (O_a += P_a V, S_a = Q_a K^T of the next
// tile, then the same for b), so that the tensor cores work for one head while the other's
// softmax runs. The probabilities never touch shared memory: each thread overwrites the scores of
// its own row in tensor memory with them (bf16, two per column) and the second product reads its
// A operand from there; products issued by one thread run in order, so the next tile's scores
// land on those columns only after the product that read them.
constexpr int PAIR_THREADS = 320;   // warp 0 producer, warp 1 MMA issuer, warps 2-5 and 6-9 the softmax warpgroups
constexpr int PAIR_SMEM = TILE_BYTES * (2 + 2 * KV_STAGES) + 1024 + 512 + TABLE_CACHE * 4;   // Q x2, K and V stages, slack, barriers, table

__global__ void __launch_bounds__(PAIR_THREADS, 1)
attention_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                              const Args args) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;                                   // [2][TILE_BYTES]
  uint8_t* k_s = q_s + 2 * TILE_BYTES;                   // [KV_STAGES][TILE_BYTES]
  uint8_t* v_s = k_s + KV_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + KV_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2 heads] the scores of a tile are in tensor memory
  uint64_t* p_full = bars + 11;       // [2 heads] the probabilities are, and the output is rescaled
  uint64_t* pv_done = bars + 13;      // [2 heads] the second product of a tile is finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* flag = tmem_slot + 1;   // [0] a wait ran out
  int* page_cache = reinterpret_cast<int*>(bars) + 128;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = args.q_heads / args.kv_heads;
  // heads run fastest and the tile list is walked backwards: later tiles of a sequence visit more keys
  const int tile_index = gridDim.y - 1 - blockIdx.y;
  const int seq = args.tile_seq[tile_index], q0 = args.tile_q0[tile_index];
  const int head0 = 2 * blockIdx.x, kv_head = head0 / group;
  const int row0 = args.cu_q[seq], q_len = args.cu_q[seq + 1] - row0, ctx = args.ctx_len[seq];
  const int n_rows = min(ROWS, q_len - q0);
  const int p_first = ctx - q_len + q0, p_last = p_first + n_rows - 1;
  const int key_lo = args.window > 0 ? max(0, p_first - args.window + 1) : 0;
  const int tile_begin = key_lo / KEYS, tile_end = p_last / KEYS + 1;
  const int q_row = row0 + q0;
  const int n_tiles = max(0, tile_end - tile_begin);
  const int* table = args.block_table + (size_t)seq * args.table_width;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&pv_done[i], 1);
    }
    flag[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;            // scores of head a, head b: 128 columns each
  const uint32_t tmem_o = tmem_base + 256;      // outputs of head a, head b
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    const int pages_per_tile = KEYS / args.page_tokens;
    if (n_tiles > 0) {
      cache_pages(page_cache, table, args.table_width, tile_begin * pages_per_tile, n_tiles * pages_per_tile, lane);
      if (lane == 0) {
        mbar_expect_tx(q_full, 2 * TILE_BYTES);
        for (int u = 0; u < 2; ++u)
          for (int half = 0; half < 2; ++half)
            tma_load_2d(q_s + u * TILE_BYTES + half * HALF_BYTES, &q_map, q_full, (head0 + u) * DIM + half * 64, q_row);
      }
      produce_kv<KV_STAGES>(&kv_map, args, k_s, v_s, k_full, k_empty, v_full, v_empty, page_cache, table, tile_begin,
                            n_tiles, kv_head, flag, 21, lane);
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc(false), idesc_o = instr_desc(true);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) { atomicCAS(&g_attn_error, 0, 22); flag[0] = 1; }
      auto issue_s = [&](int i, int u) {          // S_u = Q_u K(i)^T; K(i) has been waited for
        const int stage = i % KV_STAGES;
        const uint32_t q_addr = smem_u32(q_s + u * TILE_BYTES), k_addr = smem_u32(k_s + stage * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < DIM / 16; ++ks) {
          const uint32_t off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          umma_bf16(tmem_s + u * 128, desc_k_major(q_addr + off), desc_k_major(k_addr + off), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[u]);
        if (u == 1) umma_commit(&k_empty[stage]);
      };
      if (ok) {
        ok = mbar_wait(&k_full[0], 0);
        if (!ok) { atomicCAS(&g_attn_error, 0, 23); flag[0] = 1; }
      }
      if (ok) {
        fence_after_sync();
        issue_s(0, 0);
        issue_s(0, 1);
      }
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int stage = i % KV_STAGES;
        for (int u = 0; u < 2 && ok; ++u) {
          if (!mbar_wait(&p_full[u], i & 1) || (u == 0 && !mbar_wait(&v_full[stage], (i / KV_STAGES) & 1))) {
            atomicCAS(&g_attn_error, 0, 24); flag[0] = 1; ok = false; break;
          }
          fence_after_sync();
          const uint32_t v_addr = smem_u32(v_s + stage * TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < KEYS / 16; ++ks)       // 16 keys: 8 columns of packed probabilities, 16 rows of V
            umma_bf16_ts(tmem_o + u * 128, tmem_s + u * 128 + ks * 8, desc_mn_major(v_addr + ks * 16 * 128), idesc_o,
                         (i > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&pv_done[u]);
          if (u == 1) umma_commit(&v_empty[stage]);
          if (i + 1 < n_tiles) {
            if (u == 0 && !mbar_wait(&k_full[(i + 1) % KV_STAGES], ((i + 1) / KV_STAGES) & 1)) {
              atomicCAS(&g_attn_error, 0, 25); flag[0] = 1; ok = false; break;
            }
            fence_after_sync();
            issue_s(i + 1, u);
          }
        }
      }
    }
  } else {
    // ---------------- softmax and epilogue: warpgroup u owns head u, one query row per thread
    const int u = (warp - 2) >> 2;
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t my_s = tmem_s + u * 128 + lane_addr, my_o = tmem_o + u * 128 + lane_addr;
    const int p_row = p_first + row;                          // rows past n_rows are ballast
    const float c = args.scale_log2;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int tile = tile_begin + i, stage = i % KV_STAGES;
      const int key0 = tile * KEYS;
      if (!mbar_wait(&s_full[u], i & 1)) { atomicCAS(&g_attn_error, 0, 26); flag[0] = 1; ok = false; break; }
      fence_after_sync();
      const bool masked = key0 + KEYS - 1 > p_first || key0 < key_lo || args.window > 0;
      float s[KEYS];
      {
        uint32_t raw[64];
        tmem_ld64_nowait(my_s, raw);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 64; ++e) s[e] = __uint_as_float(raw[e]);
        tmem_ld64_nowait(my_s + 64, raw);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 64; ++e) s[64 + e] = __uint_as_float(raw[e]);
      }
      if (masked) {
#pragma unroll
        for (int e = 0; e < KEYS; ++e) {
          const int key = key0 + e;
          const bool seen = key <= p_row && key >= key_lo && (args.window <= 0 || p_row - key < args.window);
          if (!seen) s[e] = -INFINITY;
        }
      }
      const float tile_max = row_max(s);
      // the reference maximum only moves when the true one has outgrown it by 2^8 (see the kernel above)
      const bool grow = (tile_max - m_ref) * c > RESCALE_THRESHOLD || (m_ref == -INFINITY && tile_max > -INFINITY);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      const float m_new = grow ? tile_max : m_ref;
      const float factor = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_new) * c);
      const float neg_base = (m_new == -INFINITY) ? 0.f : -m_new * c;
      float part_sum[4] = {0.f, 0.f, 0.f, 0.f};           // four chains of additions side by side
      // exponentials, 32 scores at a time: 16 columns of packed probabilities over the row's own scores
#pragma unroll
      for (int ch = 0; ch < KEYS / 32; ++ch) {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float a = fast_exp2(fmaf(s[ch * 32 + 2 * e], c, neg_base));
          const float b = fast_exp2(fmaf(s[ch * 32 + 2 * e + 1], c, neg_base));
          part_sum[e & 3] += a + b;
          const __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
          w[e] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        tmem_st16_nowait(my_s + ch * 16, w);
      }
      const float tile_sum = (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
      l_sum = l_sum * factor + tile_sum;
      m_ref = m_new;
      if (any_grow && i > 0) {
        // the previous product of this head must be finished before its accumulator is touched
        if (!mbar_wait(&pv_done[u], (i - 1) & 1)) { atomicCAS(&g_attn_error, 0, 27); flag[0] = 1; ok = false; break; }
        fence_after_sync();
#pragma unroll
        for (int ch = 0; ch < DIM / 16; ++ch) {
          float v[16];
          tmem_ld16(my_o + ch * 16, v);
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] *= factor;
          tmem_st16(my_o + ch * 16, v);
        }
      }
      // V rows of keys outside the context may hold anything: zero them (0 x NaN would be NaN).
      // Both warpgroups do it, each before its own product is released.
      const int limit = p_last + 1;
      if (key0 + KEYS > limit || key0 < key_lo) {
        if (!mbar_wait(&v_full[stage], (i / KV_STAGES) & 1)) { atomicCAS(&g_attn_error, 0, 28); flag[0] = 1; ok = false; break; }
        const int key = key0 + row;
        if (key >= limit || key < key_lo) {
          uint8_t* vrow = v_s + stage * TILE_BYTES + row * 128;
#pragma unroll
          for (int chunk = 0; chunk < 8; ++chunk) {
            *reinterpret_cast<uint4*>(vrow + chunk * 16) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vrow + HALF_BYTES + chunk * 16) = make_uint4(0, 0, 0, 0);
          }
        }
        fence_async_smem();
      }
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[u]);
    }

    // ---- the head's result: wait for its last product, read the row, divide, store
    if (ok && n_tiles > 0) {
      if (!mbar_wait(&pv_done[u], (n_tiles - 1) & 1)) { atomicCAS(&g_attn_error, 0, 29); flag[0] = 1; ok = false; }
      fence_after_sync();
    }
    if (ok) {
      // tensor-memory loads are warp-wide: every lane reads its row, rows of the tile only are stored
      const bool valid = row < n_rows;
      bf16* dst = args.out + ((size_t)(q_row + (valid ? row : 0)) * args.q_heads + head0 + u) * DIM;
      const float inv = 1.0f / l_sum;
#pragma unroll
      for (int ch = 0; ch < DIM / 16; ++ch) {
        float v[16];
        if (n_tiles > 0) {
          tmem_ld16(my_o + ch * 16, v);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0.f;
        }
        if (!valid) continue;
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * e] * inv, v[2 * e + 1] * inv);
          w[e] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        reinterpret_cast<uint4*>(dst + ch * 16)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(dst + ch * 16)[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }

  // ---------------- teardown
  fence_before_sync();
  __syncthreads();
  if (flag[0]) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies in flight land
    __syncthreads();
  }
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

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

void configure_once() {      // once per device: the attribute belongs to the device that is current
  static LbPerDeviceOnce once;
  if (!once.first()) return;
  cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  cudaFuncSetAttribute(attention_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
}

// q as a 2-D bf16 matrix [rows, cols] with rows `stride` elements apart: box 64 columns x 128 rows
bool make_q_map(CUtensorMap* map, const void* q, long rows, long cols, long stride) {
  auto encode = encode_fn();
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)ROWS};
  cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

// Whether the tensor-core kernel takes these sizes.
LB_EXPORT int lb_attention_tcgen05_supports(int q_heads, int kv_heads, int dim, int page_tokens) {
  return dim == DIM && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads / kv_heads <= ROWS && page_tokens >= 8 &&
         page_tokens % 8 == 0 && KEYS % page_tokens == 0;
}

// The tensor map of one cache group's pool [planes = layers * 2, pages, kv_heads, page_tokens, dim]
// (bf16, contiguous), written to `out` (128 bytes, 64-byte aligned storage is the caller's). One map
// serves every layer and both K and V: the plane is a coordinate.
LB_EXPORT int lb_attention_tcgen05_pool_map(void* out, const void* pool, long planes, long pages, int kv_heads,
                                            int page_tokens, int dim) {
  auto encode = encode_fn();
  if (!encode || dim != DIM) return LB_ERR_SIZE;
  if ((uintptr_t)pool % 16) return LB_ERR_ALIGN;
  cuuint64_t dims[5] = {(cuuint64_t)dim, (cuuint64_t)page_tokens, (cuuint64_t)kv_heads, (cuuint64_t)pages, (cuuint64_t)planes};
  cuuint64_t strides[4] = {(cuuint64_t)dim * 2, (cuuint64_t)page_tokens * dim * 2, (cuuint64_t)kv_heads * page_tokens * dim * 2,
                           (cuuint64_t)pages * kv_heads * page_tokens * dim * 2};
  cuuint32_t box[5] = {64, (cuuint32_t)page_tokens, 1, 1, 1};
  cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  CUtensorMap map;
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(pool), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return LB_ERR_SIZE;
  memcpy(out, &map, sizeof(map));
  return 0;
}

// The device address of the error word, so that a caller's own kernel can read it along with its
// results instead of synchronising for it (null if it cannot be had).
LB_EXPORT void* lb_attention_tcgen05_status_address() {
  void* address = nullptr;
  if (cudaGetSymbolAddress(&address, g_attn_error) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  return address;
}

LB_EXPORT int lb_attention_tcgen05_status() {
  int code = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&code, g_attn_error, sizeof(int)) != cudaSuccess) return -100;
  if (code) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  return code;
}

// Prompt portions: tiles of 128 queries (tile_seq, tile_q0), grid (query heads, tiles).
LB_EXPORT int lb_attention_tcgen05_prefill(const void* q, long q_rows, const void* pool_map, int layer, void* out,
                                           const int* block_table, int table_width, const int* cu_q, const int* ctx_len,
                                           const int* tile_seq, const int* tile_q0, int n_tiles, int q_heads, int kv_heads,
                                           int dim, int page_tokens, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!lb_attention_tcgen05_supports(q_heads, kv_heads, dim, page_tokens) || n_tiles > 65535) return LB_ERR_SIZE;
  if ((uintptr_t)q % 16) return LB_ERR_ALIGN;
  configure_once();
  CUtensorMap q_map, kv_map;
  if (!make_q_map(&q_map, q, q_rows, (long)q_heads * dim, (long)q_heads * dim)) return LB_ERR_ALIGN;
  memcpy(&kv_map, pool_map, sizeof(kv_map));
  Args args{(bf16*)out, block_table, table_width, cu_q, ctx_len, tile_seq, tile_q0, q_heads, kv_heads, page_tokens, window,
            2 * layer, scale * 1.4426950408889634f};
  int code;
  if ((q_heads / kv_heads) % 2 == 0)    // two heads of a KV head per block
    code = lb_launch(attention_tcgen05_pair_kernel, dim3(q_heads / 2, n_tiles), dim3(PAIR_THREADS), (size_t)PAIR_SMEM, stream,
                     q_map, kv_map, args);
  else
    code = lb_launch(attention_tcgen05_kernel, dim3(q_heads, n_tiles), dim3(THREADS), (size_t)SMEM_BYTES, stream,
                     q_map, kv_map, args);
  return code ? code : lb_last_error();
}
