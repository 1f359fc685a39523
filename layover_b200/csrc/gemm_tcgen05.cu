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
//                          each writes a 32-bit partial tile to scratch memory and then adds up
//                          its share of the tile's columns over all splits in split order (a
//                          fixed order, so the result does not depend on timing).
//
// Two kernels share the PTX wrappers, descriptors and epilogue stores:
//   many tokens: persistent blocks of six warps, one per SM. Warp 0 lane 0 issues TMA loads through
//     a ring of stages, warp 1 lane 0 issues the MMAs into one of two accumulators in tensor memory
//     and frees stages with tcgen05.commit, warps 2-5 run the epilogue of the other accumulator.
//     Whole rounds of tiles are dealt one tile per block; the tiles left over are split along K so
//     that the last round keeps every SM busy, and the blocks of a tile then add up the partial
//     tiles together, each its share of the columns, in split order.
//     From 512 tokens on the same kernel runs on PAIRS of blocks (clusters of two, cta_group::2):
//     a pair takes tiles of 256 tokens x 256 weight rows, each block stages half of either operand
//     and keeps the accumulator rows of its own 128 tokens; the q/k/v projection of 128-dim heads
//     then also norms, rotates and stores the heads in its epilogue.
//   few tokens: one tile (or one K range of a tile) per block of four warps, two blocks per SM; the
//     block that arrives last at the tile's counter adds the partial tiles in split order.
// Every wait (on an mbarrier, or on sibling blocks) is bounded: when a limit runs out the block
// records an error code, lets copies in flight land, frees its tensor memory and returns;
// `lb_gemm_tcgen05_status` reports it.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int SMEM_BUDGET = 200 * 1024;

__device__ int g_gemm_error = 0;   // 0 = ok; a wait ran out in 1 the producer, 2 the MMA issuer, 3 the epilogue, 4 the split sum

// Persistent blocks, each over its share of the work. Shared memory holds a ring of stages
// (one 128 x 64 tile of the 128-row operand and one BN x 64 tile of the other); tensor memory holds
// two accumulators, so the epilogue of one tile overlaps the MMAs of the next.
constexpr int SMALL_THREADS = 128;

// With the SwiGLU epilogue the weight's rows come in blocks of 128: 64 gate rows of features
// f .. f + 63, then the 64 up rows of the same features. A product tile then holds both halves of
// every feature it covers, and the kernel writes silu(gate) * up, half as many columns as the
// product has: C[token, feature].
// The few-token orientation keeps two blocks on an SM (half the shared memory each), so that a
// weight matrix with about as many tiles as SMs, or one split in two, still runs in one wave.
template <int BN> struct SmallTile {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BUDGET = SMEM_BUDGET / 2;
  static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
  static constexpr int BLOCKS_PER_SM = 2;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int RECV_BYTES = BM * BN * 4;         // what a block of a cluster receives: its rows of every split
  static constexpr int SMEM_CLUSTER = SMEM + RECV_BYTES;
};

// The few-token kernel: D[i, j] = sum_k W[i, k] X[j, k] with 128 weight rows i per block, C[j, i] = D.
// One tile (or one K range of a tile) per block, two blocks per SM, four warps that all join the
// epilogue: for these short streams it starts and ends a few microseconds sooner than the
// persistent kernel below.
// CLUSTER: the `splits` blocks of a tile are one cluster (grid z = cluster z = splits, a power of
// two). Block r owns rows r * 128 / splits .. of the tile: every block sends those rows of its
// accumulator into r's shared memory, and after the cluster's barrier r adds them in split order
// and stores them. No scratch memory, fence, counter or last block: the sum starts one barrier
// after the slowest block's last MMA.
// EPI 2 (with CLUSTER, bf16, 128-dim heads): the product is the fused q/k/v projection of at most BN
// tokens. Block r owns tokens r * BN / splits ..: it receives every row of those tokens, and per
// token and head does what the per-head norm kernel does (RMSNorm of q and k heads, rotation,
// every rounding in the same place and the sum of squares in the same order, so the bits agree),
// then writes q to its buffer and k and v to their page. The projection never reaches memory.
template <int BN, typename OutT, int EPI, bool CLUSTER = false>
__global__ void __launch_bounds__(SMALL_THREADS, SmallTile<BN>::BLOCKS_PER_SM)
gemm_fewtoken_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OutT* __restrict__ C, long ldc, int rows_a, int rows_b, int K, int splits,
                    float* __restrict__ partials, unsigned* __restrict__ counters, const HeadsEpilogue he) {
  using T = SmallTile<BN>;
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
      tma_load_2d(tiles_a + i * T::A_BYTES, &map_a, &full[i], (kb_begin + i) * BK, m0);
    }
    pdl_wait();
    for (int i = 0; i < early; ++i) {
      tma_load_2d(tiles_b + i * T::B_BYTES, &map_b, &full[i], (kb_begin + i) * BK, n0);
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
  // The q/k/v epilogue gives every warp whole tokens: lane l holds features l, l + 32 (the low half of
  // the head) and l + 64, l + 96 (their partners in the high half). What it needs per token (cos,
  // sin, slot) and per feature (norm weight) does not depend on the product: it is read now, under
  // the main loop, not token by token afterwards.
  constexpr int OWNED_PER_WARP = 2;               // a block owns at most BN / 2 = 8 tokens, a warp every fourth
  float pre_cs[OWNED_PER_WARP][2], pre_sn[OWNED_PER_WARP][2], pre_w[4] = {0.f, 0.f, 0.f, 0.f};
  int pre_slot[OWNED_PER_WARP];
  if (CLUSTER && EPI == 2) {
    const int tokens_per = BN / splits, head = blockIdx.x;
    const bool is_q = head < he.q_heads, is_k = !is_q && head < he.q_heads + he.kv_heads;
    const float* w = is_q ? he.q_norm_w : (is_k ? he.k_norm_w : nullptr);
    if (w) {
#pragma unroll
      for (int e = 0; e < 4; ++e) pre_w[e] = w[lane + 32 * e];
    }
#pragma unroll
    for (int i = 0; i < OWNED_PER_WARP; ++i) {
      const int jj = warp + 4 * i, token = blockIdx.y * BN + (int)blockIdx.z * tokens_per + jj;
      pre_cs[i][0] = pre_cs[i][1] = 1.f; pre_sn[i][0] = pre_sn[i][1] = 0.f; pre_slot[i] = 0;
      if (jj < tokens_per && token < rows_b) {
        if (w) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            pre_cs[i][e] = round_bf16(he.rope_table[((size_t)token * 2) * 64 + lane + 32 * e]);
            pre_sn[i][e] = round_bf16(he.rope_table[((size_t)token * 2 + 1) * 64 + lane + 32 * e]);
          }
        }
        if (!is_q) pre_slot[i] = he.slot_map[token];
      }
    }
  }
  const bool ready = mbar_wait(tmem_full, 0);
  if (!ready) { atomicCAS(&g_gemm_error, 0, 3); flag[0] = 1; }
  fence_after_sync();
  const int row = warp * 32 + lane;                       // row of the 128-row side
  const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
  const int valid_cols = min(BN, rows_b - n0);
  const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
  float* my_partial = (partials && !CLUSTER) ? partials + ((size_t)tile_id * splits + split) * BN * BM : nullptr;

  if (CLUSTER && EPI == 2) {
    const int tokens_per = BN / splits;
    float* recv = reinterpret_cast<float*>(smem + T::STAGES * T::STAGE_BYTES + 256);   // [splits][128][tokens_per]
    // send: this row's values of the tokens that a block owns are neighbours there
    for (int c = 0; c < BN; c += 16) {
      if (c >= valid_cols) break;                                    // the same for the whole block
      float v[16];
      if (ready) {
        tmem_ld16(lane_base + c, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
      if (tokens_per % 4 == 0) {
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          const int j = c + i;
          if (j < valid_cols)
            lb_store_remote4(lb_map_to_rank(smem_u32(recv + ((size_t)split * BM + row) * tokens_per + j % tokens_per),
                                            (uint32_t)(j / tokens_per)), v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int j = c + i;
          if (j < valid_cols)
            lb_store_remote(lb_map_to_rank(smem_u32(recv + ((size_t)split * BM + row) * tokens_per + j % tokens_per),
                                           (uint32_t)(j / tokens_per)), v[i]);
        }
      }
    }
    lb_cluster_barrier();        // reached by every thread, also after a wait that ran out
    const int head = blockIdx.x;
    const bool is_q = head < he.q_heads, is_k = !is_q && head < he.q_heads + he.kv_heads;
#pragma unroll
    for (int i = 0; i < OWNED_PER_WARP; ++i) {
      const int jj = warp + 4 * i, token = n0 + (int)lb_cluster_rank() * tokens_per + jj;
      if (jj >= tokens_per || token >= rows_b) break;                // the same for the whole warp
      float x[4];                                                    // features lane, +32, +64, +96
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float sum = 0.f;
        for (int sp = 0; sp < splits; ++sp) sum += recv[((size_t)sp * BM + lane + 32 * e) * tokens_per + jj];
        x[e] = round_bf16(sum);                                      // the projection's own rounding
      }
      if (is_q || is_k) {
        // The sum of squares in the order of the per-head kernel: eight lanes of eight (low, high)
        // pairs each, one after the other, then a butterfly over the eight partial sums. Pair
        // (x[0], x[2]) is pair lane % 8 of partial sum lane / 8, pair (x[1], x[3]) of partial sum lane / 8 + 4.
        const float sq_a = lb_square_pair(x[0], x[2]), sq_b = lb_square_pair(x[1], x[3]);
        float part_a = 0.f, part_b = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          part_a += __shfl_sync(0xffffffffu, sq_a, (lane & 24) + j);
          part_b += __shfl_sync(0xffffffffu, sq_b, (lane & 24) + j);
        }
        const float pair_sum = part_a + part_b;                      // p[g] + p[g + 4], g = lane / 8
        const float ss = (__shfl_sync(0xffffffffu, pair_sum, 0) + __shfl_sync(0xffffffffu, pair_sum, 16)) +
                         (__shfl_sync(0xffffffffu, pair_sum, 8) + __shfl_sync(0xffffffffu, pair_sum, 24));
        const float inv = 1.0f / sqrtf(ss / (float)BM + he.eps);
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = round_bf16(pre_w[e] * round_bf16(x[e] * inv));
        // rotate_half(x) = (-hi, lo): each product and the sum round to bfloat16
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float cs = pre_cs[i][e], sn = pre_sn[i][e];
          x[e] = round_bf16(round_bf16(y[e] * cs) + round_bf16(-y[e + 2] * sn));
          x[e + 2] = round_bf16(round_bf16(y[e + 2] * cs) + round_bf16(y[e] * sn));
        }
      }
      bf16* dst;
      if (is_q) {
        dst = he.q_out + ((size_t)token * he.q_heads + head) * BM;
      } else {
        const int kvh = is_k ? head - he.q_heads : head - he.q_heads - he.kv_heads;
        const size_t page = pre_slot[i] / he.page_tokens, within = pre_slot[i] % he.page_tokens;
        dst = (is_k ? he.k_pool : he.v_pool) + ((page * he.kv_heads + kvh) * he.page_tokens + within) * BM;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) dst[lane + 32 * e] = __float2bfloat16_rn(x[e]);
    }
  } else if (CLUSTER) {
    const int rows_per = BM / splits;
    float* recv = reinterpret_cast<float*>(smem + T::STAGES * T::STAGE_BYTES + 256);   // [splits][rows_per][BN]
    const uint32_t owner = (uint32_t)(row / rows_per);
    const uint32_t dst = lb_map_to_rank(smem_u32(recv + ((size_t)split * rows_per + row % rows_per) * BN), owner);
    for (int c = 0; c < BN; c += 16) {
      float v[16];
      if (ready) {
        tmem_ld16(lane_base + c, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 16; i += 4) lb_store_remote4(dst + (c + i) * 4, v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    lb_cluster_barrier();        // reached by every thread, also after a wait that ran out
    const int first_row = m0 + (int)lb_cluster_rank() * rows_per;
    for (int idx = threadIdx.x; idx < rows_per * valid_cols; idx += SMALL_THREADS) {
      const int j = idx / rows_per, r = idx % rows_per;
      float sum = 0.f;
      for (int sp = 0; sp < splits; ++sp) sum += recv[((size_t)sp * rows_per + r) * BN + j];
      if (first_row + r < rows_a) store_one<OutT>(C + (size_t)(n0 + j) * ldc + first_row + r, sum);
    }
  } else if (ready) {
    for (int c = 0; c < BN; c += 16) {
      if (c >= valid_cols) break;                           // uniform over the block
      float v[16];
      tmem_ld16(lane_base + c, v);
      if (splits > 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (c + i < valid_cols) my_partial[(size_t)(c + i) * BM + row] = v[i];
      } else if (EPI == 1) {
        // rows 0..63 of the tile are gate rows, rows 64..127 the up rows of the same features: the
        // upper half hands its values over through shared memory (the ring is drained by now)
        float* handover = reinterpret_cast<float*>(tiles_a);           // [64][17]
        if (row >= 64) {
#pragma unroll
          for (int i = 0; i < 16; ++i) handover[(row - 64) * 17 + i] = v[i];
        }
        __syncthreads();
        if (row < 64 && m0 + row < rows_a) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c + i < valid_cols)
              store_one<OutT>(C + (size_t)(n0 + c + i) * ldc + (m0 >> 1) + row, swiglu_bf16(v[i], handover[row * 17 + i]));
        }
        __syncthreads();
      } else {
        if (m0 + row < rows_a) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c + i < valid_cols) store_one<OutT>(C + (size_t)(n0 + c + i) * ldc + m0 + row, v[i]);
        }
      }
    }
  }

  if (!CLUSTER && splits > 1) {
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
              store_one<OutT>(C + (size_t)(n0 + j0 + u) * ldc + m0 + row, sum[u]);
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


// ------------------------------------------------------------------ the persistent kernel
// The few-token orientation asks for two blocks per SM (half the shared memory each): a weight
// matrix with about as many tiles as SMs then still runs in one round.
// PAIR: two blocks of a cluster work as one MMA unit on a tile of 256 rows x BN columns; each block
// stages its own 128 rows and its own half of the BN columns' operand, a third fewer bytes into
// each SM per product than a block on its own, and so more stages in the same memory.
template <int BN, bool SWAP, bool PAIR = false> struct Tile {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BLOCKS_PER_SM = SWAP ? 2 : 1;
  static constexpr int BUDGET = SMEM_BUDGET / BLOCKS_PER_SM;   // a pair's seventh stage fits in 227 KB, and measured no faster
  static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
  static constexpr int ACC_COLS = BN < 16 ? 16 : BN;          // columns of one accumulator
  static constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ +
                              (PAIR ? 1024 : 0) /* norm weights of the q/k/v epilogue */;
};

// How the output tiles are dealt to the blocks. Tiles are numbered with the 128-row side fastest.
// `full` rounds give block b the whole tile round * blocks + b. The `rem` tiles left over form a
// last round in which each tile is cut into `last_splits` ranges of K, one per block; a block
// whose range is not the whole K writes a 32-bit partial tile to scratch memory and the block that
// has a partial tile then adds up its own share of the tile's columns, in split order.
struct Schedule {
  int tiles_m, tiles, full, rem, last_splits, total_kb;
};

struct Segment {
  int tile, split, splits, kb_begin, kb_end;
};

__device__ __forceinline__ int segment_count(const Schedule& sch, int block) {
  return sch.full + ((sch.rem > 0 && block < sch.rem * sch.last_splits) ? 1 : 0);
}
__device__ __forceinline__ Segment segment_at(const Schedule& sch, int block, int blocks, int j) {
  Segment seg;
  if (j < sch.full) {
    seg.tile = j * blocks + block; seg.split = 0; seg.splits = 1; seg.kb_begin = 0; seg.kb_end = sch.total_kb;
  } else {
    seg.tile = sch.full * blocks + block % sch.rem;
    seg.split = block / sch.rem;
    seg.splits = sch.last_splits;
    seg.kb_begin = (int)((long)sch.total_kb * seg.split / seg.splits);
    seg.kb_end = (int)((long)sch.total_kb * (seg.split + 1) / seg.splits);
  }
  return seg;
}

constexpr int EPILOGUE_WARPS = 4;
constexpr int PERSISTENT_THREADS = (2 + EPILOGUE_WARPS) * 32;
// the q/k/v epilogue (EPI 2) does more per value, so two warps share each quarter of the accumulator's
// lanes, one per head of the tile
__host__ __device__ constexpr int epilogue_warps(int epi) { return epi == 2 ? 2 * EPILOGUE_WARPS : EPILOGUE_WARPS; }
__host__ __device__ constexpr int persistent_threads(int epi) { return (2 + epilogue_warps(epi)) * 32; }

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// D[i, j] = sum_k Aop[i, k] Bop[j, k], i on the 128-row side. SWAP false: C[i, j] = D; true: C[j, i] = D.
// PAIR (never with SWAP): the grid is clusters of two blocks along x. What the schedule calls a block
// is a pair, and a tile has 256 rows: block `rank` of the pair stages rows 128 rank .. of the A side
// and rows BN / 2 * rank .. of the B side, all copies report to the leader's `full` barriers, the
// leader (rank 0) issues MMAs of M = 256 whose commits arrive on the `empty` and `acc_full` barriers
// of both blocks, both blocks' epilogues arrive on the leader's `acc_empty`, and each block's
// epilogue handles its own 128 rows like a tile of its own (with a scratch slot of its own when K
// is split).
template <int BN, bool SWAP, typename OutT, int EPI, bool PAIR = false>
__global__ void __launch_bounds__(persistent_threads(EPI), Tile<BN, SWAP, PAIR>::BLOCKS_PER_SM)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OutT* __restrict__ C, long ldc, int rows_a, int rows_b, const Schedule sch,
                    float* __restrict__ partials, unsigned* __restrict__ counters, bool vector_ok, const HeadsEpilogue he) {
  static_assert(!(PAIR && SWAP), "pairs of blocks serve the many-token orientation");
  static_assert(EPI != 2 || (PAIR && BN == 256 && sizeof(OutT) == 2), "the q/k/v epilogue takes a pair's 256-column tiles of bfloat16");
  using T = Tile<BN, SWAP, PAIR>;
  constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles_a = smem;
  uint8_t* tiles_b = smem + T::STAGES * T::A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + T::STAGES * T::STAGE_BYTES);
  uint64_t* empty = full + T::STAGES;
  uint64_t* acc_full = empty + T::STAGES;     // [2] the MMAs of an accumulator are done
  uint64_t* acc_empty = acc_full + 2;         // [2] the epilogue has read an accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* flag = tmem_slot + 1;    // [0] a wait ran out, [1] this block is the last of its tile
  float* norm_w = reinterpret_cast<float*>(smem + T::STAGES * T::STAGE_BYTES + 256);   // EPI 2: [2][128] q and k norm weights

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = PAIR ? (int)lb_cluster_rank() : 0;                // 0: the block that issues the MMAs
  const int block = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int blocks = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int n_segments = segment_count(sch, block);

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], (PAIR ? 2 : 1) * epilogue_warps(EPI)); }
    flag[0] = 0; flag[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair(tmem_slot, T::TMEM_COLS);
    else tmem_alloc(tmem_slot, T::TMEM_COLS);
  }
  if (EPI == 2) {      // weights, which no kernel writes: no need to wait for the kernel before
    for (int i = threadIdx.x; i < 2 * BM; i += blockDim.x) norm_w[i] = i < BM ? he.q_norm_w[i] : he.k_norm_w[i - BM];
  }
  fence_before_sync();
  if (PAIR) lb_cluster_barrier();      // neither block signals the other's barriers before they exist
  else __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (PAIR && warp == 0) {
    if (lane == 0) {
      // ---------------- producer of a pair: this block's rows of both operands, reported to the leader
      const uint32_t leader_full = lb_map_to_rank(smem_u32(full), 0);
      pdl_wait();
      int it = 0;
      for (int j = 0; j < n_segments && !flag[0]; ++j) {
        const Segment seg = segment_at(sch, block, blocks, j);
        const int m0 = (seg.tile % sch.tiles_m) * TILE_ROWS + rank * BM;
        const int n0 = (seg.tile / sch.tiles_m) * BN + rank * (BN / 2);
        for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb, ++it) {
          const int s = it % T::STAGES;
          const uint32_t phase = (it / T::STAGES) & 1;
          if (it >= T::STAGES && !mbar_wait(&empty[s], phase ^ 1)) { atomicCAS(&g_gemm_error, 0, 1); flag[0] = 1; break; }
          if (rank == 0) mbar_expect_tx(&full[s], 2 * T::STAGE_BYTES);
          tma_load_2d_pair(tiles_a + s * T::A_BYTES, &map_a, leader_full + 8u * s, kb * BK, m0);
          tma_load_2d_pair(tiles_b + s * T::B_BYTES, &map_b, leader_full + 8u * s, kb * BK, n0);
        }
      }
    }
  } else if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer. Weights are written by no kernel, so the first ring of weight
      // tiles is requested before waiting for the kernel that produces the activations.
      int it = 0;                       // K blocks issued so far, over all segments
      bool waited = false;
      for (int j = 0; j < n_segments && !flag[0]; ++j) {
        const Segment seg = segment_at(sch, block, blocks, j);
        const int m0 = (seg.tile % sch.tiles_m) * BM, n0 = (seg.tile / sch.tiles_m) * BN;
        for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb, ++it) {
          const int s = it % T::STAGES;
          const uint32_t phase = (it / T::STAGES) & 1;
          if (it >= T::STAGES && !waited) {
            // the ring is full of weight tiles: now the activations are needed
            pdl_wait();
            waited = true;
            int back = 0;               // replay the first ring's activation tiles
            for (int jj = 0; jj <= j && back < T::STAGES; ++jj) {
              const Segment early = segment_at(sch, block, blocks, jj);
              const int em0 = (early.tile % sch.tiles_m) * BM, en0 = (early.tile / sch.tiles_m) * BN;
              for (int ekb = early.kb_begin; ekb < early.kb_end && back < T::STAGES; ++ekb, ++back) {
                if (SWAP) tma_load_2d(tiles_b + back * T::B_BYTES, &map_b, &full[back], ekb * BK, en0);
                else tma_load_2d(tiles_a + back * T::A_BYTES, &map_a, &full[back], ekb * BK, em0);
              }
            }
          }
          if (it >= T::STAGES && !mbar_wait(&empty[s], phase ^ 1)) { atomicCAS(&g_gemm_error, 0, 1); flag[0] = 1; break; }
          mbar_expect_tx(&full[s], T::STAGE_BYTES);
          if (!waited) {                // only the weight half for now
            if (SWAP) tma_load_2d(tiles_a + s * T::A_BYTES, &map_a, &full[s], kb * BK, m0);
            else tma_load_2d(tiles_b + s * T::B_BYTES, &map_b, &full[s], kb * BK, n0);
          } else {
            tma_load_2d(tiles_a + s * T::A_BYTES, &map_a, &full[s], kb * BK, m0);
            tma_load_2d(tiles_b + s * T::B_BYTES, &map_b, &full[s], kb * BK, n0);
          }
        }
      }
      if (!waited) {                    // fewer K blocks than stages: same replay, after the wait
        pdl_wait();
        int back = 0;
        for (int jj = 0; jj < n_segments && back < T::STAGES; ++jj) {
          const Segment early = segment_at(sch, block, blocks, jj);
          const int em0 = (early.tile % sch.tiles_m) * BM, en0 = (early.tile / sch.tiles_m) * BN;
          for (int ekb = early.kb_begin; ekb < early.kb_end && back < T::STAGES; ++ekb, ++back) {
            if (SWAP) tma_load_2d(tiles_b + back * T::B_BYTES, &map_b, &full[back], ekb * BK, en0);
            else tma_load_2d(tiles_a + back * T::A_BYTES, &map_a, &full[back], ekb * BK, em0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc = instr_desc(BN, TILE_ROWS);
      int it = 0;
      for (int j = 0; j < n_segments && !flag[0]; ++j) {
        const Segment seg = segment_at(sch, block, blocks, j);
        const int buf = j & 1;
        if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1)) { atomicCAS(&g_gemm_error, 0, 2); flag[0] = 1; break; }
        fence_after_sync();
        const uint32_t acc = tmem_base + buf * T::ACC_COLS;
        for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb, ++it) {
          const int s = it % T::STAGES;
          const uint32_t phase = (it / T::STAGES) & 1;
          if (!mbar_wait(&full[s], phase)) { atomicCAS(&g_gemm_error, 0, 2); flag[0] = 1; break; }
          fence_after_sync();
          const uint64_t a_desc = smem_desc(tiles_a + s * T::A_BYTES), b_desc = smem_desc(tiles_b + s * T::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {  // +32 bytes per K step inside the swizzled row
            if (PAIR) umma_bf16_pair(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > seg.kb_begin || k > 0) ? 1u : 0u);
            else umma_bf16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > seg.kb_begin || k > 0) ? 1u : 0u);
          }
          if (PAIR) umma_commit_pair(&empty[s], 3);
          else umma_commit(&empty[s]);
        }
        if (flag[0]) break;
        if (PAIR) umma_commit_pair(&acc_full[buf], 3);
        else umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue: four warps, each owning the accumulator lanes 32 (warp % 4) ..
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                    // row of the 128-row side
    pdl_wait();   // the stores below touch memory that earlier kernels may still be reading
    for (int j = 0; j < n_segments; ++j) {
      const Segment seg = segment_at(sch, block, blocks, j);
      const int m0 = (seg.tile % sch.tiles_m) * TILE_ROWS + rank * BM, n0 = (seg.tile / sch.tiles_m) * BN;
      const int buf = j & 1;
      if (!mbar_wait(&acc_full[buf], (j >> 1) & 1)) { atomicCAS(&g_gemm_error, 0, 3); flag[0] = 1; break; }
      fence_after_sync();
      const uint32_t lane_base = tmem_base + buf * T::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const int valid_cols = min(BN, rows_b - n0);
      // index among the last round's tiles; each block of a pair has a partial tile of its own
      const int slot = PAIR ? 2 * (seg.tile - sch.full * blocks) + rank : seg.tile - sch.full * blocks;
      float* my_partial = seg.splits > 1 ? partials + ((size_t)slot * seg.splits + seg.split) * BN * BM : nullptr;
      if (EPI == 2) {
        // The fused q/k/v projection (never split along K): the tile's 256 columns are two heads of
        // 128, one for each of the two warps that share this quarter of the lanes, and this thread
        // holds one token's row of its head. It does what the per-head norm kernel does, every
        // rounding in the same place and the sum of squares in the same order (that kernel's eight
        // lanes of eight (low, high) pairs, then its butterfly), so the bits agree: RMSNorm and
        // rotation of q and k heads, q to its buffer, k and v to their page. The accumulator is read
        // twice (sum, then values) instead of keeping 128 values in registers.
        const int token = m0 + row;
        const bool live = token < rows_a;
        const int half = (warp - 2) >> 2;
        if (half * 128 < valid_cols) {
          const int head = (n0 >> 7) + half;
          const bool is_q = head < he.q_heads, is_k = !is_q && head < he.q_heads + he.kv_heads;
          const float* w = is_q ? norm_w : (is_k ? norm_w + BM : nullptr);
          const uint32_t col0 = lane_base + half * 128;
          float inv = 0.f;
          if (w) {
            float part[8];
#pragma unroll
            for (int c = 0; c < 64; c += 16) {
              float lo[16], hi[16];
              tmem_ld16_two(col0 + c, col0 + 64 + c, lo, hi);
#pragma unroll
              for (int g = 0; g < 2; ++g) {
                float ss = 0.f;
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) ss += lb_square_pair(round_bf16(lo[8 * g + jj]), round_bf16(hi[8 * g + jj]));
                part[(c >> 3) + g] = ss;
              }
            }
            const float ss = ((part[0] + part[4]) + (part[2] + part[6])) + ((part[1] + part[5]) + (part[3] + part[7]));
            inv = 1.0f / sqrtf(ss / (float)BM + he.eps);
          }
          bf16* dst = nullptr;
          if (live) {
            if (is_q) {
              dst = he.q_out + ((size_t)token * he.q_heads + head) * BM;
            } else {
              const int slot_id = he.slot_map[token];
              const int kvh = is_k ? head - he.q_heads : head - he.q_heads - he.kv_heads;
              const size_t page = slot_id / he.page_tokens, within = slot_id % he.page_tokens;
              dst = (is_k ? he.k_pool : he.v_pool) + ((page * he.kv_heads + kvh) * he.page_tokens + within) * BM;
            }
          }
          const float* cos_row = he.rope_table + (size_t)(live ? token : 0) * 2 * 64;
#pragma unroll
          for (int c = 0; c < 64; c += 16) {
            float4 cs4[4], sn4[4];
            if (w) {       // asked for before the accumulator's values, so that both are on their way together
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                cs4[i] = __ldg(reinterpret_cast<const float4*>(cos_row + c) + i);
                sn4[i] = __ldg(reinterpret_cast<const float4*>(cos_row + 64 + c) + i);
              }
            }
            float lo[16], hi[16];
            tmem_ld16_two(col0 + c, col0 + 64 + c, lo, hi);
#pragma unroll
            for (int i = 0; i < 16; ++i) { lo[i] = round_bf16(lo[i]); hi[i] = round_bf16(hi[i]); }   // the projection's own rounding
            if (w) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float cs[4] = {cs4[i].x, cs4[i].y, cs4[i].z, cs4[i].w}, sn[4] = {sn4[i].x, sn4[i].y, sn4[i].z, sn4[i].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int d = 4 * i + e;
                  const float yl = round_bf16(w[c + d] * round_bf16(lo[d] * inv));
                  const float yh = round_bf16(w[64 + c + d] * round_bf16(hi[d] * inv));
                  const float cc = round_bf16(cs[e]), sv = round_bf16(sn[e]);
                  // rotate_half(x) = (-hi, lo): each product and the sum round to bfloat16
                  lo[d] = round_bf16(round_bf16(yl * cc) + round_bf16(-yh * sv));
                  hi[d] = round_bf16(round_bf16(yh * cc) + round_bf16(yl * sv));
                }
              }
            }
            if (dst) {
              store_row16<bf16>(dst + c, lo);
              store_row16<bf16>(dst + 64 + c, hi);
            }
          }
        }
      }
      if (EPI == 1 && seg.splits == 1) {
        // columns come as [64 gate | 64 up] per 128: one thread holds both halves of its token's
        // features and writes 64 activations per 128 columns
        for (int half = 0; half * 128 < valid_cols; ++half) {
#pragma unroll
          for (int cc = 0; cc < 64; cc += 16) {
            float g[16], u[16];
            tmem_ld16(lane_base + half * 128 + cc, g);
            tmem_ld16(lane_base + half * 128 + 64 + cc, u);
            if (m0 + row < rows_a) {
#pragma unroll
              for (int i = 0; i < 16; ++i) g[i] = swiglu_bf16(g[i], u[i]);
              OutT* dst = C + (size_t)(m0 + row) * ldc + (n0 >> 1) + half * 64 + cc;
              if (vector_ok) {
                store_row16<OutT>(dst, g);
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) store_one<OutT>(dst + i, g[i]);
              }
            }
          }
        }
      }
      for (int c = 0; c < BN && !(EPI == 1 && seg.splits == 1) && EPI != 2; c += 16) {
        if (c >= valid_cols) break;                           // uniform over the block
        float v[16];
        tmem_ld16(lane_base + c, v);
        if (seg.splits > 1) {
          // four columns of a row side by side: 16-byte stores here, 16-byte loads in the sum
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<float4*>(my_partial)[(size_t)((c >> 2) + i) * BM + row] =
                make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
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
      // the accumulator may be overwritten now
      fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(lb_map_to_rank(smem_u32(&acc_empty[buf]), 0));
        else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
      }

      if (seg.splits > 1) {
        // Every block of the tile adds up its own share of the columns, over all splits in split
        // order, once all partial tiles are there. All blocks of a launch are resident at once
        // (one per SM, at most as many as SMs), so waiting for the siblings is safe; the wait is
        // bounded all the same. counters[2 slot] counts partial tiles written, [2 slot + 1] counts
        // blocks that finished reading; the last reader puts both back to zero.
        volatile unsigned* written = counters + 2 * slot;
        __threadfence();
        epilogue_sync();
        if (threadIdx.x == 64) {
          atomicAdd(const_cast<unsigned*>(written), 1u);
          bool ok = false;
          for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
            if (*written >= (unsigned)seg.splits) { ok = true; break; }
            __nanosleep(32);
          }
          if (!ok) { atomicCAS(&g_gemm_error, 0, 4); flag[0] = 1; }
          flag[1] = ok ? 1u : 0u;
        }
        epilogue_sync();
        if (flag[1]) {
          __threadfence();
          const float4* tile_partials = reinterpret_cast<const float4*>(partials + (size_t)slot * seg.splits * BN * BM);
          const int quads = (valid_cols + 3) >> 2;                      // groups of four columns
          const int share = (quads + seg.splits - 1) / seg.splits;
          const int q_begin = seg.split * share, q_end = min(quads, q_begin + share);
          if (EPI == 1) {
            // shares of OUTPUT quads: output quad o of a 128-column half h sums gate quad
            // 32 h + o and up quad 32 h + 16 + o over the splits, then combines them
            const int out_quads = valid_cols >> 3;
            const int out_share = (out_quads + seg.splits - 1) / seg.splits;
            const int o_begin = seg.split * out_share, o_end = min(out_quads, o_begin + out_share);
            if (m0 + row < rows_a) {
              for (int oq = o_begin; oq < o_end; ++oq) {
                const int gq = (oq >> 4) * 32 + (oq & 15), uq = gq + 16;
                float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
#pragma unroll 4
                for (int s0 = 0; s0 < seg.splits; ++s0) {
                  const float4 pg = tile_partials[((size_t)s0 * (BN / 4) + gq) * BM + row];
                  const float4 pu = tile_partials[((size_t)s0 * (BN / 4) + uq) * BM + row];
                  g.x += pg.x; g.y += pg.y; g.z += pg.z; g.w += pg.w;
                  u.x += pu.x; u.y += pu.y; u.z += pu.z; u.w += pu.w;
                }
                OutT* dst = C + (size_t)(m0 + row) * ldc + (n0 >> 1) + oq * 4;
                store_one<OutT>(dst, swiglu_bf16(g.x, u.x));
                store_one<OutT>(dst + 1, swiglu_bf16(g.y, u.y));
                store_one<OutT>(dst + 2, swiglu_bf16(g.z, u.z));
                store_one<OutT>(dst + 3, swiglu_bf16(g.w, u.w));
              }
            }
          } else if (m0 + row < rows_a) {
            for (int q0 = q_begin; q0 < q_end; q0 += 4) {
              float4 sum[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int s0 = 0; s0 < seg.splits; s0 += 4) {
                float4 part[4][4];
#pragma unroll
                for (int ds = 0; ds < 4; ++ds)
#pragma unroll
                  for (int u = 0; u < 4; ++u)
                    part[ds][u] = (s0 + ds < seg.splits && q0 + u < q_end)
                                      ? tile_partials[((size_t)(s0 + ds) * (BN / 4) + q0 + u) * BM + row]
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int ds = 0; ds < 4; ++ds)
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    sum[u].x += part[ds][u].x; sum[u].y += part[ds][u].y;
                    sum[u].z += part[ds][u].z; sum[u].w += part[ds][u].w;
                  }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                if (q0 + u >= q_end) continue;
                const int col = (q0 + u) * 4;
                const float vals[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
                if (!SWAP && vector_ok && col + 4 <= valid_cols) {
                  OutT* dst = C + (size_t)(m0 + row) * ldc + n0 + col;
                  if (sizeof(OutT) == 2) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(vals[0], vals[1]), hi = __floats2bfloat162_rn(vals[2], vals[3]);
                    uint2 w;
                    w.x = *reinterpret_cast<const uint32_t*>(&lo);
                    w.y = *reinterpret_cast<const uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst) = w;
                  } else {
                    *reinterpret_cast<float4*>(dst) = sum[u];
                  }
                } else {
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (col + e < valid_cols) {
                      if (SWAP) store_one<OutT>(C + (size_t)(n0 + col + e) * ldc + m0 + row, vals[e]);
                      else store_one<OutT>(C + (size_t)(m0 + row) * ldc + n0 + col + e, vals[e]);
                    }
                  }
                }
              }
            }
          }
        }
        epilogue_sync();
        if (threadIdx.x == 64 && flag[1]) {
          const unsigned finished = atomicAdd(counters + 2 * slot + 1, 1u);
          if (finished == (unsigned)seg.splits - 1) {   // everyone has read: ready for the next launch
            counters[2 * slot + 1] = 0;
            __threadfence();
            *written = 0;
          }
        }
      }
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
  if (PAIR) lb_cluster_barrier();       // the other block may still signal this one's barriers until here
  if (warp == 1) {
    fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, T::TMEM_COLS);
    else tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
// What the caller knows about the product; the launcher turns it into a schedule.
struct Problem {
  int rows_a, rows_b, K, bn;
  bool swap;
  int sm_count, max_splits;
  float* scratch;
  long scratch_floats;
  unsigned* counters;
  int n_counters;
};

template <int BN, bool SWAP, typename OutT, int EPI = 0>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, void* C, long ldc, const Problem& pb, bool vector_ok,
           cudaStream_t stream) {
  using T = Tile<BN, SWAP>;
  auto kernel = gemm_tcgen05_kernel<BN, SWAP, OutT, EPI>;
  static int blocks_per_sm = 0;      // how many blocks of this kernel an SM really holds (the same on every B200)
  static LbPerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM) != cudaSuccess)
      return lb_last_error();
    int fit = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, kernel, PERSISTENT_THREADS, T::SMEM) != cudaSuccess || fit < 1)
      return lb_last_error() ? lb_last_error() : LB_ERR_SIZE;
    blocks_per_sm = fit < T::BLOCKS_PER_SM ? fit : T::BLOCKS_PER_SM;
  }
  // Blocks that split a tile wait for one another, so a launch never has more blocks than the GPU
  // holds at once.
  const int slots = pb.sm_count * blocks_per_sm;
  Schedule sch;
  sch.tiles_m = (pb.rows_a + BM - 1) / BM;
  sch.tiles = sch.tiles_m * ((pb.rows_b + BN - 1) / BN);
  sch.total_kb = (pb.K + BK - 1) / BK;
  // A split costs a partial tile to write, a fence, a counter and a longer sum; wider token tiles
  // make the partial tiles bigger. Measured on 2560..9728-wide weights: 8 splits of a 20-tile
  // matrix beat 15, and 128-token tiles want 2. One block per SM streams a weight matrix at close
  // to full bandwidth, so splitting aims at one block per SM, not at every slot.
  // Token tiles of 128 (prompt portions): the left-over round of 2560-wide outputs (160 tiles on 148
  // SMs) ran 86 us with 4 splits, 80 us with 8 and 12, 82 us with 16 on a 9728-deep product.
  int cap = SWAP ? (BN <= 16 ? 8 : (BN <= 32 ? 4 : 2)) : 8;
  if (pb.max_splits > 0) cap = pb.max_splits;
  if (!pb.scratch || !pb.counters) cap = 1;
  int blocks;
  if (sch.tiles >= slots) {
    blocks = slots;
    sch.full = sch.tiles / blocks;
    sch.rem = sch.tiles % blocks;
  } else {
    blocks = sch.tiles;              // grows below when the tiles are split
    sch.full = 0;
    sch.rem = sch.tiles;
  }
  sch.last_splits = 1;
  if (sch.rem > 0) {
    int splits = sch.rem < pb.sm_count ? (pb.sm_count + sch.rem - 1) / sch.rem : 1;
    if (splits > cap) splits = cap;
    if (splits > sch.total_kb / 4) splits = sch.total_kb / 4;       // at least four K blocks per split
    if (splits > slots / sch.rem) splits = slots / sch.rem;
    const long per_split = (long)sch.rem * BN * BM;
    if (splits > 1 && per_split * splits > pb.scratch_floats) splits = (int)(pb.scratch_floats / per_split);
    if (splits > 1 && 2 * sch.rem > pb.n_counters) splits = 1;
    if (splits < 1) splits = 1;
    sch.last_splits = splits;
    if (sch.full == 0) blocks = sch.rem * splits;
  }
  float* partials = sch.last_splits > 1 ? pb.scratch : nullptr;
  const int code = lb_launch(kernel, dim3(blocks), dim3(PERSISTENT_THREADS), (size_t)T::SMEM, stream, map_a, map_b,
                             (OutT*)C, ldc, pb.rows_a, pb.rows_b, sch, partials, pb.counters, vector_ok, HeadsEpilogue{});
  return code ? code : lb_last_error();
}

// The many-token product on pairs of blocks (`cta_group::2`), tiles of 256 tokens x 256 weight rows.
// Returns -1 when this GPU holds no cluster of two such blocks (nothing is launched then).
// LAYOVER_B200_GEMM_PAIR=0 keeps every product on single blocks.
static inline bool lb_gemm_pair_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("LAYOVER_B200_GEMM_PAIR");
    return !(v && v[0] == '0');
  }();
  return enabled;
}

template <typename OutT, int EPI = 0>
int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, void* C, long ldc, const Problem& pb, bool vector_ok,
                cudaStream_t stream, const HeadsEpilogue& he = HeadsEpilogue{}) {
  constexpr int BN = 256;
  using T = Tile<BN, false, true>;
  auto kernel = gemm_tcgen05_kernel<BN, false, OutT, EPI, true>;
  static int pairs_resident = 0;      // clusters of two that the GPU holds at once (the same on every B200)
  static LbPerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM) != cudaSuccess)
      return lb_last_error();
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2 * pb.sm_count);
    probe.blockDim = dim3(persistent_threads(EPI));
    probe.dynamicSmemBytes = T::SMEM;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;       // the two blocks of an MMA pair are neighbours along x
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    probe.attrs = attribute;
    probe.numAttrs = 1;
    int fit = 0;
    if (cudaOccupancyMaxActiveClusters(&fit, kernel, &probe) != cudaSuccess) { cudaGetLastError(); fit = 0; }
    pairs_resident = fit;
  }
  // Blocks that split a tile wait for one another, so a launch never has more pairs than the GPU
  // holds at once.
  const int slots = pairs_resident < pb.sm_count / 2 ? pairs_resident : pb.sm_count / 2;
  if (slots < 1) return -1;
  Schedule sch;
  sch.tiles_m = (pb.rows_a + 2 * BM - 1) / (2 * BM);
  sch.tiles = sch.tiles_m * ((pb.rows_b + BN - 1) / BN);
  sch.total_kb = (pb.K + BK - 1) / BK;
  int cap = pb.max_splits > 0 ? pb.max_splits : 8;
  if (!pb.scratch || !pb.counters || EPI == 2) cap = 1;      // the q/k/v epilogue needs whole sums in one place
  int pairs;
  if (sch.tiles >= slots) {
    pairs = slots;
    sch.full = sch.tiles / pairs;
    sch.rem = sch.tiles % pairs;
  } else {
    pairs = sch.tiles;
    sch.full = 0;
    sch.rem = sch.tiles;
  }
  sch.last_splits = 1;
  if (sch.rem > 0) {
    int splits = slots / sch.rem;
    if (splits > cap) splits = cap;
    if (splits > sch.total_kb / 4) splits = sch.total_kb / 4;       // at least four K blocks per split
    const long per_split = (long)sch.rem * 2 * BN * BM;              // each block of a pair has a partial tile
    if (splits > 1 && per_split * splits > pb.scratch_floats) splits = (int)(pb.scratch_floats / per_split);
    if (splits > 1 && 4 * sch.rem > pb.n_counters) splits = 1;
    if (splits < 1) splits = 1;
    sch.last_splits = splits;
    if (sch.full == 0) pairs = sch.rem * splits;
  }
  float* partials = sch.last_splits > 1 ? pb.scratch : nullptr;
  const int code = lb_launch_cluster_dims(kernel, dim3(2 * pairs), dim3(persistent_threads(EPI)), (size_t)T::SMEM, stream,
                                          dim3(2, 1, 1), map_a, map_b, (OutT*)C, ldc, pb.rows_a, pb.rows_b, sch, partials,
                                          pb.counters, vector_ok, he);
  return code ? code : lb_last_error();
}

template <int BN, typename OutT, int EPI = 0>
int launch_fewtoken(const CUtensorMap& map_a, const CUtensorMap& map_b, void* C, long ldc, const Problem& pb,
                    cudaStream_t stream) {
  using T = SmallTile<BN>;
  auto kernel = gemm_fewtoken_kernel<BN, OutT, EPI>;
  static LbPerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM) != cudaSuccess)
      return lb_last_error();
  }
  const int tiles = (pb.rows_a + BM - 1) / BM, total_kb = (pb.K + BK - 1) / BK;
  int splits = 1;
  if (EPI == 0 && pb.scratch && pb.counters && tiles <= pb.n_counters && tiles < pb.sm_count) {
    // One block per SM streams a weight matrix at close to full bandwidth, and every further
    // split adds a partial tile to write, a fence, a counter and a longer sum, which at these
    // sizes cost more than the extra blocks win (measured on 2560..9728-wide weights: 8 splits
    // of a 20-tile matrix beat 15; a 152-tile matrix is fastest unsplit). Wider token tiles
    // make the partial tiles bigger, so they split less.
    const int cap = BN <= 16 ? 8 : (BN <= 32 ? 4 : 2);
    splits = (pb.sm_count + tiles - 1) / tiles;
    if (splits > cap) splits = cap;
    if (splits > total_kb / 4) splits = total_kb / 4;         // at least four K blocks per split
    if (pb.max_splits > 0 && splits > pb.max_splits) splits = pb.max_splits;
    const long per_split = (long)tiles * BN * BM;
    if (splits > 1 && per_split * splits > pb.scratch_floats) splits = (int)(pb.scratch_floats / per_split);
    if (splits < 1) splits = 1;
  }
  dim3 grid(tiles, (pb.rows_b + BN - 1) / BN, splits);
  if constexpr (EPI == 0 && BN <= 32) {
    if (splits > 1 && splits <= 8 && (splits & (splits - 1)) == 0 && lb_cluster_reduce_enabled()) {
      // the K ranges of a tile as one cluster: partial sums travel through distributed shared memory
      auto cluster_kernel = gemm_fewtoken_kernel<BN, OutT, EPI, true>;
      static LbPerDeviceOnce cluster_configured;
      if (cluster_configured.first()) {
        if (cudaFuncSetAttribute(cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_CLUSTER) != cudaSuccess)
          return lb_last_error();
      }
      const int code = lb_launch_cluster(cluster_kernel, grid, dim3(SMALL_THREADS), (size_t)T::SMEM_CLUSTER, stream,
                                         (unsigned)splits, map_a, map_b, (OutT*)C, ldc, pb.rows_a, pb.rows_b, pb.K,
                                         splits, (float*)nullptr, (unsigned*)nullptr, HeadsEpilogue{});
      return code ? code : lb_last_error();
    }
  }
  const int code = lb_launch(kernel, grid, dim3(SMALL_THREADS), (size_t)T::SMEM, stream, map_a, map_b, (OutT*)C, ldc,
                             pb.rows_a, pb.rows_b, pb.K, splits, splits > 1 ? pb.scratch : (float*)nullptr, pb.counters,
                             HeadsEpilogue{});
  return code ? code : lb_last_error();
}

// The fused q/k/v projection of at most 16 tokens with 128-dim heads: returns 1 when the sizes do
// not allow it (nothing is launched then and the caller runs the product and the norm kernel).
int launch_heads(const CUtensorMap& map_a, const CUtensorMap& map_b, const Problem& pb, const HeadsEpilogue& he,
                 cudaStream_t stream) {
  constexpr int BN = 16;
  using T = SmallTile<BN>;
  const int tiles = (pb.rows_a + BM - 1) / BM, total_kb = (pb.K + BK - 1) / BK;
  int splits = (pb.sm_count + tiles - 1) / tiles;
  if (splits > 8) splits = 8;
  if (splits > total_kb / 4) splits = total_kb / 4;           // at least four K blocks per split
  while (splits & (splits - 1)) splits &= splits - 1;         // down to a power of two
  if (splits < 2 || !lb_cluster_reduce_enabled()) return 1;
  auto kernel = gemm_fewtoken_kernel<BN, bf16, 2, true>;
  static LbPerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_CLUSTER) != cudaSuccess)
      return lb_last_error();
  }
  dim3 grid(tiles, 1, splits);
  const int code = lb_launch_cluster(kernel, grid, dim3(SMALL_THREADS), (size_t)T::SMEM_CLUSTER, stream, (unsigned)splits,
                                     map_a, map_b, (bf16*)nullptr, 0L, pb.rows_a, pb.rows_b, pb.K, splits, (float*)nullptr,
                                     (unsigned*)nullptr, he);
  return code ? code : lb_last_error();
}
}  // namespace

// The device address of the error word, so that a caller's own kernel can read it along with its
// results instead of synchronising for it (null if it cannot be had).
LB_EXPORT void* lb_gemm_tcgen05_status_address() {
  void* address = nullptr;
  if (cudaGetSymbolAddress(&address, g_gemm_error) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  return address;
}

// Writes the error word from the host: a drill for the path that reports a wait that ran out (a test
// sets a code, runs a step and expects the engine to refuse the step's tokens and to recover).
LB_EXPORT int lb_gemm_tcgen05_set_status(int code) {
  return cudaMemcpyToSymbol(g_gemm_error, &code, sizeof(int)) == cudaSuccess ? 0 : -100;
}

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
// never split. `sm_count` sizes the grid; `max_splits` > 0 caps the splitting. `epilogue` 1: W's rows
// come as blocks of 64 gate rows + 64 up rows and C[M, N / 2] = silu(gate) * up (bfloat16 only).
LB_EXPORT int lb_gemm_tcgen05(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K, long lda,
                              long ldw, long ldc, float* scratch, long scratch_floats, unsigned* counters,
                              int n_counters, int sm_count, int max_splits, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (epilogue != 0 && epilogue != 1) return LB_ERR_SIZE;
  if (epilogue == 1 && (N % 128 != 0 || out_dtype != LB_BF16)) return LB_ERR_SIZE;   // blocks of 64 gate + 64 up rows
  if (!lb_gemm_tcgen05_supports(A, W, K, lda, ldw)) return LB_ERR_ALIGN;
  if (out_dtype != LB_BF16 && out_dtype != LB_F32) return LB_ERR_DTYPE;
  if (sm_count < 1) sm_count = 1;
  const bool swap = M <= 128;
  CUtensorMap map_a, map_b;
  int bn, rows_a, rows_b;
  if (swap) {
    bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    rows_a = N; rows_b = M;
    if (!make_map(&map_a, W, N, K, ldw, BM) || !make_map(&map_b, A, M, K, lda, bn)) return LB_ERR_ALIGN;
  } else {
    // 256-wide tiles: half the shared-memory traffic per flop of 128-wide ones, which measured
    // slower at every size even with two blocks per SM
    bn = N > 128 ? 256 : 128;
    rows_a = M; rows_b = N;
    if (!make_map(&map_a, A, M, K, lda, BM) || !make_map(&map_b, W, N, K, ldw, bn)) return LB_ERR_ALIGN;
  }
  const Problem pb{rows_a, rows_b, K, bn, swap, sm_count, max_splits, scratch, scratch_floats, counters, n_counters};
  const int elem = out_dtype == LB_BF16 ? 2 : 4;
  const bool vector_ok = ((uintptr_t)C % 16 == 0) && ((ldc * elem) % 16 == 0);
  // Prompt portions of 512 tokens and more on 256-wide weights: pairs of blocks on tiles of 256 x 256
  if (!swap && bn == 256 && M >= 512 && lb_gemm_pair_enabled()) {
    CUtensorMap map_half;
    if (make_map(&map_half, W, N, K, ldw, 128)) {
      int code;
      if (epilogue == 1) code = launch_pair<bf16, 1>(map_a, map_half, C, ldc, pb, vector_ok, stream);
      else if (out_dtype == LB_BF16) code = launch_pair<bf16>(map_a, map_half, C, ldc, pb, vector_ok, stream);
      else code = launch_pair<float>(map_a, map_half, C, ldc, pb, vector_ok, stream);
      if (code != -1) return code;
    }
  }
#define LB_GEMM_CASE(BN_, SWAP_)                                                                       \
  if (bn == BN_ && swap == SWAP_) {                                                                    \
    if (out_dtype == LB_BF16) return launch<BN_, SWAP_, bf16>(map_a, map_b, C, ldc, pb, vector_ok, stream); \
    return launch<BN_, SWAP_, float>(map_a, map_b, C, ldc, pb, vector_ok, stream);                     \
  }
#define LB_FEWTOKEN_CASE(BN_)                                                                          \
  if (bn == BN_ && swap) {                                                                             \
    if (out_dtype == LB_BF16) return launch_fewtoken<BN_, bf16>(map_a, map_b, C, ldc, pb, stream);     \
    return launch_fewtoken<BN_, float>(map_a, map_b, C, ldc, pb, stream);                              \
  }
  if (epilogue == 1) {
    if (swap) {
      if (bn == 16) return launch_fewtoken<16, bf16, 1>(map_a, map_b, C, ldc, pb, stream);
      if (bn == 32) return launch_fewtoken<32, bf16, 1>(map_a, map_b, C, ldc, pb, stream);
      if (bn == 64) return launch_fewtoken<64, bf16, 1>(map_a, map_b, C, ldc, pb, stream);
      return launch_fewtoken<128, bf16, 1>(map_a, map_b, C, ldc, pb, stream);
    }
    if (bn == 128) return launch<128, false, bf16, 1>(map_a, map_b, C, ldc, pb, vector_ok, stream);
    return launch<256, false, bf16, 1>(map_a, map_b, C, ldc, pb, vector_ok, stream);
  }
  // 32..128 tokens and a weight with fewer 128-row tiles than SMs: the persistent kernel, whose
  // blocks add up the partial tiles together, takes 8 splits well (measured: 11 us against 18 us
  // for a 2560 x 4096 weight at 64 tokens); weights with more tiles run unsplit in the one-tile kernel.
  if (swap && bn >= 32 && (N + BM - 1) / BM < sm_count && scratch && counters) {
    Problem split = pb;
    if (split.max_splits <= 0) split.max_splits = 8;
    if (out_dtype == LB_BF16) {
      if (bn == 32) return launch<32, true, bf16>(map_a, map_b, C, ldc, split, vector_ok, stream);
      if (bn == 64) return launch<64, true, bf16>(map_a, map_b, C, ldc, split, vector_ok, stream);
      return launch<128, true, bf16>(map_a, map_b, C, ldc, split, vector_ok, stream);
    }
    if (bn == 32) return launch<32, true, float>(map_a, map_b, C, ldc, split, vector_ok, stream);
    if (bn == 64) return launch<64, true, float>(map_a, map_b, C, ldc, split, vector_ok, stream);
    return launch<128, true, float>(map_a, map_b, C, ldc, split, vector_ok, stream);
  }
  LB_FEWTOKEN_CASE(16)
  LB_FEWTOKEN_CASE(32)
  LB_FEWTOKEN_CASE(64)
  LB_FEWTOKEN_CASE(128)
#undef LB_FEWTOKEN_CASE
  LB_GEMM_CASE(128, false)
  LB_GEMM_CASE(256, false)
#undef LB_GEMM_CASE
  return LB_ERR_SIZE;
}

// The q/k/v projection of `M` tokens fused with the per-head norm, the rotation and the page
// write: W [(q_heads + 2 kv_heads) * 128, K] stacked q, k, v; what `lb_gemm_tcgen05` followed by the
// per-head norm kernel would leave in q_out and the pools, bit for bit. Up to 16 tokens run in the
// few-token kernel (clusters along K), 512 and more on pairs of blocks (a thread of the epilogue
// holds a token's whole head). Returns 0 when launched, 1 when these sizes are not taken (head size
// other than 128, 17..511 tokens, too few K blocks to split, clusters or pairs switched off):
// nothing has been launched then.
LB_EXPORT int lb_gemm_qkv_heads(const void* A, const void* W, int M, int K, long lda, long ldw, int q_heads, int kv_heads,
                                int head_dim, const float* q_norm_w, const float* k_norm_w, const float* rope_table,
                                int n_freq, const int* slot_map, void* q_out, void* k_pool, void* v_pool, int page_tokens,
                                float eps, int sm_count, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (head_dim != BM || (M > 16 && M < 512) || n_freq * 2 != head_dim || !q_norm_w || !k_norm_w || !rope_table ||
      !slot_map || !q_out || !k_pool || !v_pool || q_heads < 1 || kv_heads < 1 || page_tokens < 1)
    return 1;
  if (!lb_gemm_tcgen05_supports(A, W, K, lda, ldw)) return 1;
  if (sm_count < 1) sm_count = 1;
  const int rows = (q_heads + 2 * kv_heads) * head_dim;
  CUtensorMap map_a, map_b;
  if (M >= 512) {
    if (!lb_gemm_pair_enabled() || rows <= 128) return 1;
    if (!make_map(&map_a, A, M, K, lda, BM) || !make_map(&map_b, W, rows, K, ldw, 128)) return 1;
    const Problem many{M, rows, K, 256, false, sm_count, 1, nullptr, 0, nullptr, 0};
    const HeadsEpilogue he{q_norm_w, k_norm_w, rope_table, slot_map, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool,
                           q_heads, kv_heads, page_tokens, eps};
    const int code = launch_pair<bf16, 2>(map_a, map_b, nullptr, 0L, many, false, stream, he);
    return code == -1 ? 1 : code;
  }
  if (!make_map(&map_a, W, rows, K, ldw, BM) || !make_map(&map_b, A, M, K, lda, 16)) return 1;
  const Problem pb{rows, M, K, 16, true, sm_count, 0, nullptr, 0, nullptr, 0};
  const HeadsEpilogue he{q_norm_w, k_norm_w, rope_table, slot_map, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool,
                         q_heads, kv_heads, page_tokens, eps};
  return launch_heads(map_a, map_b, pb, he, stream);
}
