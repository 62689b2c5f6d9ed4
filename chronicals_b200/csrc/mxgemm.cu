// Block-scaled MXFP8 GEMM on the 5th-generation tensor cores:
//
//   C[M, N] (bf16) = sum_k  (Aq[m, k] * 2^(SFA[m, k/32] - 127)) * (Bq[n, k] * 2^(SFB[n, k/32] - 127))   (+ bias[n])
//
// Aq, Bq are e4m3 (or e5m2) bytes, both K-major; SFA, SFB are e8m0 scale bytes, one per 32 elements
// of K (OCP microscaling).  The scales are applied by the tensor core itself:
// `tcgen05.mma.kind::mxf8f6f4.block_scale` reads them from tensor memory, where `tcgen05.cp` has put
// them from shared memory, so the fp32 accumulator in TMEM holds the exactly scaled products and no
// dequantised copy of either operand ever exists.
//
// Scale layout.  The quantiser writes the scales already in the order the hardware wants: for every
// 128 rows x 4 scale blocks (= 128 elements of K) one 512-byte atom,
//     byte (r % 32) * 16 + ((r / 32) % 4) * 4 + (kb % 4),
// atoms ordered [row block][k block / 4].  One pipeline stage (128 rows x 128 bytes of K) therefore
// needs exactly one contiguous atom per operand: a 512-byte bulk copy brings it to shared memory and
// one `tcgen05.cp.32x128b.warpx4` spreads it over 4 TMEM columns (lane = r % 32 in each of the four
// lane quarters, column = r / 32, byte within the column = kb % 4, selected per MMA by the scale-id
// fields of the instruction descriptor).
//
// Kernel: persistent, 192 threads.  warp 0 = TMA producer (A tile, B tile, two scale atoms per
// stage), warp 1 = one thread issues `tcgen05.cp` x2 and 4 MMAs (K = 32 each) per stage into one of
// two 128-column accumulators, warps 2-5 = epilogue (`tcgen05.ld`, + bias, bf16 stores).  Every
// stage has its own scale columns in TMEM, so a copy for stage s+1 never overwrites scales that
// MMAs of stage s still read.  Every wait is bounded.
//
// Replaces the reference's simulated FP8 linear (quantise, dequantise, bf16 matmul:
// chronicals/utils/fp8_deepseek.py:612-760, chronicals/utils/fp8_utils.py) with real block-scaled
// tensor-core arithmetic.
#include "common.cuh"
#include "host_common.h"

namespace cbmx {

using cb::bf16;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BKB = 128;          // bytes (= fp8 elements) of K per stage: one 128-byte swizzle row
constexpr int UMMA_K = 32;        // elements per MMA
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BKB;  // 16 KB
constexpr int B_BYTES = BN * BKB;  // 16 KB
constexpr int SF_BYTES = 512;      // one scale atom
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;
constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
constexpr int SMEM_TOTAL = BAR_OFFSET + 256 + 1024;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SF_COL0 = 2 * BN;      // scale columns start after the two accumulators
constexpr uint32_t SF_COLS_PER_STAGE = 8;  // 4 for A, 4 for B

struct Args {
  int M, N, K;
  int num_m_blocks, num_n_tiles, num_tiles;
  int sf_kb4;                 // scale atoms per row block (= ceil(K / 128))
  bf16* C;
  long long ldc;
  const bf16* bias;
  const unsigned char* sfa;   // packed scale atoms of A: [ceil(M/128)][sf_kb4][512]
  const unsigned char* sfb;   // packed scale atoms of B: [ceil(N/128)][sf_kb4][512]
  int* status;
};

// Instruction descriptor of kind::mxf8f6f4 with block scaling: a/b format at bits 7 and 10
// (0 = e4m3, 1 = e5m2), N >> 3 at bit 17, scale format e8m0 at bit 23, M >> 4 at bit 24; the scale
// ids (which byte of the 32-bit scale column this MMA uses) sit at bits 4 (B) and 29 (A).
__host__ __device__ constexpr uint32_t idesc_mx(int m, int n, int afmt, int bfmt) {
  return (static_cast<uint32_t>(afmt) << 7) | (static_cast<uint32_t>(bfmt) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory descriptor without swizzle for the scale copy: 32 rows of 16 bytes, 8-row core
// matrices 128 bytes apart.
__device__ __forceinline__ uint64_t sf_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((128u >> 4) & 0x3FFF) << 32;   // stride between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version for sm_100
  return d;
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void umma_mx_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier (both addresses and the size
// are multiples of 16 bytes)
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(cb::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(cb::smem_u32(bar))
               : "memory");
}

template <int AFMT, int BFMT>
__global__ void __launch_bounds__(THREADS, 1)
mxgemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Args g) {
  using namespace cb;
  constexpr uint32_t IDESC = idesc_mx(BM, BN, AFMT, BFMT);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull + a, 1);
      mbar_init(tempty + a, 4);
    }
    mbar_fence_init();
    *abort_flag = (g.status[0] != 0) ? 1 : 0;
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  __syncthreads();
  if (*abort_flag) return;  // poisoned by an earlier timeout: uniform early exit, nothing allocated yet
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (g.K + BKB - 1) / BKB;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < g.num_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile % g.num_m_blocks;
        const int nt = tile / g.num_m_blocks;
        const unsigned char* sfa_row = g.sfa + static_cast<size_t>(m_blk) * g.sf_kb4 * SF_BYTES;
        const unsigned char* sfb_row = g.sfb + static_cast<size_t>(nt) * g.sf_kb4 * SF_BYTES;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* st = smem + stage * STAGE_BYTES;
          mbar_expect_tx(full + stage, STAGE_BYTES);
          tma_load_2d(st, &tmA, full + stage, kb * BKB, m_blk * BM);
          tma_load_2d(st + A_BYTES, &tmB, full + stage, kb * BKB, nt * BN);
          bulk_load(st + A_BYTES + B_BYTES, sfa_row + static_cast<size_t>(kb) * SF_BYTES, SF_BYTES, full + stage);
          bulk_load(st + A_BYTES + B_BYTES + SF_BYTES, sfb_row + static_cast<size_t>(kb) * SF_BYTES, SF_BYTES,
                    full + stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- scale copies + MMA issue
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tile_cnt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < g.num_tiles && ok; tile += gridDim.x, ++tile_cnt) {
        const uint32_t acc = tile_cnt & 1u;
        const uint32_t acc_phase = (tile_cnt >> 1) & 1u;
        if (!mbar_wait(tempty + acc, acc_phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t a_base = st, b_base = st + A_BYTES;
          const uint32_t tsfa = tmem_base + SF_COL0 + stage * SF_COLS_PER_STAGE;
          const uint32_t tsfb = tsfa + 4;
          tmem_cp_sf(tsfa, sf_smem_desc(st + A_BYTES + B_BYTES));
          tmem_cp_sf(tsfb, sf_smem_desc(st + A_BYTES + B_BYTES + SF_BYTES));
#pragma unroll
          for (uint32_t k = 0; k < BKB / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = umma_smem_desc(b_base + k * 32, 16, 1024);
            // scale block k of this stage = byte k of the scale columns, for A and for B
            umma_mx_ss(d_tmem, adesc, bdesc, IDESC | (k << 4) | (k << 29), tsfa, tsfb, (kb != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit(empty + stage);  // frees the stage (data and scales) once the copies and MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(tfull + acc);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (4 warps, one TMEM lane quarter each)
    const int q = warp & 3;
    uint32_t tile_cnt = 0;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(g.C) & 15) == 0 && (g.ldc & 7) == 0;
    for (int tile = blockIdx.x; tile < g.num_tiles; tile += gridDim.x, ++tile_cnt) {
      const int m_blk = tile % g.num_m_blocks;
      const int nt = tile / g.num_m_blocks;
      const uint32_t acc = tile_cnt & 1u;
      const uint32_t acc_phase = (tile_cnt >> 1) & 1u;
      bool w = mbar_wait(tfull + acc, acc_phase, abort_flag, g.status, CB_ERR_WAIT_TMEM_FULL);
      w = __all_sync(0xffffffffu, w);
      if (!w) break;
      tc_fence_after();
      const int row = m_blk * BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col0 = nt * BN + c0;
        if (col0 >= g.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
        if (row < g.M) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (g.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < g.N) v[j] += __bfloat162float(g.bias[col0 + j]);
          }
          bf16* dst = g.C + static_cast<long long>(row) * g.ldc + col0;
          if (vec_ok && col0 + 32 <= g.N) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 u;
              u.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
              u.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
              u.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
              u.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
              reinterpret_cast<uint4*>(dst)[j] = u;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < g.N; ++j) dst[j] = __float2bfloat16(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty + acc);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int AFMT, int BFMT>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Args& g, cudaStream_t s) {
  auto kern = mxgemm_kernel<AFMT, BFMT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  int grid = g.num_tiles < cbhost::num_sms() ? g.num_tiles : cbhost::num_sms();
  kern<<<grid, THREADS, SMEM_TOTAL, s>>>(ta, tb, g);
  return static_cast<int>(cudaGetLastError());
}


// =====================================================================================================
// CTA-pair variant: one 256 x 192 output tile per pair of CTAs (`tcgen05.mma.cta_group::2`).
//
// With one CTA per 128 x 128 tile every 128 elements of K cost 32 KB of operand traffic per 128 x 128 x 128
// multiply-accumulates, and at FP8 rates the L2 -> shared-memory path, not the tensor core, sets the pace
// (measured: tensor pipe 37 % active).  A pair shares B: each CTA loads its own 128 rows of A and only
// 96 of the 192 rows of B (28 KB per 128 x 192 x 128), and the tensor cores of both SMs read both halves.
// The pipeline is bound by bytes in flight (shared-memory capacity over memory latency), so the ring is as deep
// as 227 KB allow: seven stages, the scale atoms packed behind the operand ring, one staging buffer per warp.
// 192 columns (not 256) because tensor memory has 512 columns per SM: two accumulators of 192 leave room
// for the scale columns (4 for A, 8 for B, four rotating sets).
//
// Each CTA needs the scales of its own 128 rows of A and of ALL 192 rows of B in its own tensor memory;
// `tcgen05.cp.cta_group::2`, issued once by the leader, copies from each CTA's own shared memory (same
// offsets) into each CTA's own tensor memory.  The B scales are packed for 192-row tiles: tile t owns two
// 512-byte atoms per 128 elements of K (rows 0-127 and 128-191 of the tile; the rest of the second atom is
// padding), addressed as ((2 t + j) * kb4 + kb) * 512.
// Roles, barriers, bounded waits and the way the pair leaves together are those of gemm2sm.cu.
constexpr int P_BN = 192;
constexpr int P_BNH = 96;
constexpr int P_STAGES = 7;
constexpr int P_A_BYTES = BM * BKB;              // 16 KB
constexpr int P_B_BYTES = P_BNH * BKB;           // 12 KB
constexpr int P_DATA_BYTES = P_A_BYTES + P_B_BYTES;            // 28 KB per stage, every stage base 1024-aligned
constexpr int P_SF_STAGE = 3 * SF_BYTES;                       // scale atoms of a stage: A, B rows 0-127, B rows 128-191
constexpr int P_TX_BYTES = P_DATA_BYTES + P_SF_STAGE;
constexpr int P_SF_OFFSET = P_STAGES * P_DATA_BYTES;           // the scale atoms sit behind the operand ring
constexpr int P_STG_OFFSET = (P_SF_OFFSET + P_STAGES * P_SF_STAGE + 1023) / 1024 * 1024;
constexpr int P_BAR_OFFSET = P_STG_OFFSET + 4 * 4096;          // epilogue staging: one 4 KB buffer per warp
constexpr int P_SMEM_TOTAL = P_BAR_OFFSET + 512 + 1024;
static_assert(P_SMEM_TOTAL <= 232448, "shared memory per CTA");
constexpr uint32_t P_SF_COL0 = 2 * P_BN;         // 384
constexpr uint32_t P_SF_SET = 12;                // columns per scale set: 4 (A) + 8 (B)

struct PairArgs {
  int M, N, K;
  int num_m_pairs, num_n_tiles, num_tiles;
  int sf_kb4;
  const bf16* bias;
  const unsigned char* sfa;   // atoms of A: [ceil(M/128)][sf_kb4][512]
  const unsigned char* sfb;   // atoms of B for 192-row tiles: [n_tiles][2][sf_kb4][512]
  int* status;
};

__device__ __forceinline__ void tmem_cp_sf_2cta(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_mx_ss_2cta(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}

template <int AFMT, int BFMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
mxgemm2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const PairArgs g) {
  using namespace cb;
  constexpr uint32_t IDESC = idesc_mx(2 * BM, P_BN, AFMT, BFMT);           // M = 256 across the pair

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + P_BAR_OFFSET);       // my stage landed
  uint64_t* peer_full = full + P_STAGES;                                   // (leader) the peer's stage landed
  uint64_t* empty = peer_full + P_STAGES;                                  // stage consumed (multicast commit)
  uint64_t* tfull = empty + P_STAGES;                                      // accumulator complete (multicast commit)
  uint64_t* tempty = tfull + 2;                                            // (leader) accumulator drained by both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(peer_full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull + a, 1);
      mbar_init(tempty + a, 8);                                            // 4 epilogue warps in each CTA
    }
    mbar_fence_init();
    *abort_flag = (g.status[0] != 0) ? 1 : 0;
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  __syncthreads();
  cluster_sync_all();                                                      // barriers of both CTAs are initialised
  // both CTAs take the LEADER's view of "poisoned by an earlier timeout", so the pair always decides alike
  const uint32_t poisoned = ld_shared_cluster_u32(mapa_u32(smem_u32(const_cast<int*>(abort_flag)), 0));
  cluster_sync_all();                                                      // nobody leaves while its flag is being read
  if (poisoned != 0) return;
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  cluster_sync_all();                                                      // both halves of the pair hold their TMEM
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (g.K + BKB - 1) / BKB;

  if (warp == 0) {
    // ------------------------------------------------------------- producer (each CTA: its A rows, its B half, scales)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < g.num_tiles && ok; t += num_pairs) {
        const int mp = t % g.num_m_pairs;
        const int nt = t / g.num_m_pairs;
        const int a_row = mp * 2 * BM + static_cast<int>(rank) * BM;
        const int b_row = nt * P_BN + static_cast<int>(rank) * P_BNH;
        const unsigned char* sfa_row = g.sfa + static_cast<size_t>(mp * 2 + static_cast<int>(rank)) * g.sf_kb4 * SF_BYTES;
        const unsigned char* sfb0 = g.sfb + static_cast<size_t>(nt) * 2 * g.sf_kb4 * SF_BYTES;
        const unsigned char* sfb1 = sfb0 + static_cast<size_t>(g.sf_kb4) * SF_BYTES;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* st = smem + stage * P_DATA_BYTES;
          uint8_t* sf = smem + P_SF_OFFSET + stage * P_SF_STAGE;
          mbar_expect_tx(full + stage, P_TX_BYTES);
          tma_load_2d(st, &tmA, full + stage, kb * BKB, a_row);
          tma_load_2d(st + P_A_BYTES, &tmB, full + stage, kb * BKB, b_row);
          bulk_load(sf, sfa_row + static_cast<size_t>(kb) * SF_BYTES, SF_BYTES, full + stage);
          bulk_load(sf + SF_BYTES, sfb0 + static_cast<size_t>(kb) * SF_BYTES, SF_BYTES, full + stage);
          bulk_load(sf + 2 * SF_BYTES, sfb1 + static_cast<size_t>(kb) * SF_BYTES, SF_BYTES, full + stage);
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (leader) {
        // --------------------------------------------------------- scale copies + MMA issue for the pair
        uint32_t tile_cnt = 0, it = 0;
        for (int t = pair; t < g.num_tiles && ok; t += num_pairs, ++tile_cnt) {
          const uint32_t acc = tile_cnt & 1u;
          const uint32_t acc_phase = (tile_cnt >> 1) & 1u;
          if (!mbar_wait(tempty + acc, acc_phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * P_BN;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            if (!mbar_wait(full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_FULL) ||
                !mbar_wait(peer_full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_PEER)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_base = smem_u32(smem + stage * P_DATA_BYTES), b_base = a_base + P_A_BYTES;
            const uint32_t sf_base = smem_u32(smem + P_SF_OFFSET + stage * P_SF_STAGE);
            const uint32_t tsfa = tmem_base + P_SF_COL0 + (it & 3u) * P_SF_SET;
            const uint32_t tsfb = tsfa + 4;
            tmem_cp_sf_2cta(tsfa, sf_smem_desc(sf_base));
            tmem_cp_sf_2cta(tsfb, sf_smem_desc(sf_base + SF_BYTES));
            tmem_cp_sf_2cta(tsfb + 4, sf_smem_desc(sf_base + 2 * SF_BYTES));
#pragma unroll
            for (uint32_t k = 0; k < BKB / UMMA_K; ++k) {
              const uint64_t adesc = umma_smem_desc(a_base + k * 32, 16, 1024);
              const uint64_t bdesc = umma_smem_desc(b_base + k * 32, 16, 1024);
              umma_mx_ss_2cta(d_tmem, adesc, bdesc, IDESC | (k << 4) | (k << 29), tsfa, tsfb,
                              (kb != 0 || k != 0) ? 1u : 0u);
            }
            umma_commit_2cta(empty + stage);      // frees this stage in both CTAs once the copies and MMAs retire
            if (++stage == P_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok) umma_commit_2cta(tfull + acc);  // accumulator complete, visible to both epilogues
        }
      } else {
        // --------------------------------------------------------- relay: tell the leader that my stage is full
        const uint32_t remote0 = mapa_u32(smem_u32(peer_full), 0);
        for (int t = pair; t < g.num_tiles && ok; t += num_pairs) {
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_FULL)) {
              ok = false;
              break;
            }
            mbar_arrive_remote(remote0 + stage * 8);
            if (++stage == P_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (4 warps, one TMEM lane quarter each)
    const int q = warp & 3;
    const uint32_t tempty_leader = mapa_u32(smem_u32(tempty), 0);
    uint8_t* stg = smem + P_STG_OFFSET + (warp - 2) * 4096;
    uint32_t tile_cnt = 0;
    for (int t = pair; t < g.num_tiles; t += num_pairs, ++tile_cnt) {
      const int mp = t % g.num_m_pairs;
      const int nt = t / g.num_m_pairs;
      const uint32_t acc = tile_cnt & 1u;
      const uint32_t acc_phase = (tile_cnt >> 1) & 1u;
      bool w = mbar_wait(tfull + acc, acc_phase, abort_flag, g.status, CB_ERR_WAIT_TMEM_FULL);
      w = __all_sync(0xffffffffu, w);
      if (!w) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * P_BN;
      const int row0w = mp * 2 * BM + static_cast<int>(rank) * BM + q * 32;
#pragma unroll 1
      for (int c0 = 0; c0 < P_BN; c0 += 64) {
        const int colbase = nt * P_BN + c0;
        if (colbase >= g.N) break;                          // uniform across the warp
        uint32_t r[64];
        tmem_ld_32x32(t_row + c0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld_32x32(t_row + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld_wait();
        if (g.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (colbase + j < g.N) r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(g.bias[colbase + j]));
        }
        if (lane == 0) tma_store_wait_read<0>();            // the previous store has read the buffer out
        __syncwarp();
        uint8_t* dstrow = stg + lane * 128;
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(r[8 * cc + 0]), __uint_as_float(r[8 * cc + 1]));
          u.y = pack_bf16x2(__uint_as_float(r[8 * cc + 2]), __uint_as_float(r[8 * cc + 3]));
          u.z = pack_bf16x2(__uint_as_float(r[8 * cc + 4]), __uint_as_float(r[8 * cc + 5]));
          u.w = pack_bf16x2(__uint_as_float(r[8 * cc + 6]), __uint_as_float(r[8 * cc + 7]));
          *reinterpret_cast<uint4*>(dstrow + ((cc ^ (lane & 7)) << 4)) = u;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0 && row0w < g.M) {                      // a box that starts past the last row has nothing to write
          tma_store_2d(&tmC, stg, colbase, row0w);
          tma_store_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(tempty + acc);
        else mbar_arrive_remote(tempty_leader + acc * 8);
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // ------------------------------------------------------------- teardown (the pair leaves together)
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

template <int AFMT, int BFMT>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const PairArgs& g, cudaStream_t s) {
  auto kern = mxgemm2sm_kernel<AFMT, BFMT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  int pairs = cbhost::num_sms() / 2;
  if (pairs > g.num_tiles) pairs = g.num_tiles;
  kern<<<2 * pairs, THREADS, P_SMEM_TOTAL, s>>>(ta, tb, tc, g);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace cbmx

extern "C" {

// Bytes of the packed scale buffer for an operand of `rows` x `K` (K a multiple of 32).
long long cb_mxgemm_sf_bytes(long long rows, int K) {
  const long long rb = (rows + 127) / 128;
  const long long kb4 = (K + 127) / 128;
  return rb * kb4 * 512;
}

// Aq [M, K], Bq [N, K]: fp8 bytes (row pitches lda, ldb bytes, multiples of 16); sfa, sfb: packed e8m0
// scale atoms (cb_mxgemm_sf_bytes each; blocks beyond K or beyond the last row hold any finite scale);
// C [M, N] bf16 (pitch ldc elements); bias [N] bf16 or null.  K must be a multiple of 32.
int cb_mxgemm(const void* Aq, const void* Bq, const void* sfa, const void* sfb, void* C, const void* bias, int M, int N,
              int K, long long lda, long long ldb, long long ldc, int a_e5m2, int b_e5m2, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || sfa == nullptr || sfb == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(sfa) & 15) != 0 || (reinterpret_cast<uintptr_t>(sfb) & 15) != 0) return -3;
  CUtensorMap ta, tb;
  int e = cbhost::make_tmap(&ta, Aq, K, M, lda, cbmx::BKB, cbmx::BM, 1);
  if (e) return e;
  e = cbhost::make_tmap(&tb, Bq, K, N, ldb, cbmx::BKB, cbmx::BN, 1);
  if (e) return e;
  cbmx::Args g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_blocks = (M + cbmx::BM - 1) / cbmx::BM;
  g.num_n_tiles = (N + cbmx::BN - 1) / cbmx::BN;
  g.num_tiles = g.num_m_blocks * g.num_n_tiles;
  g.sf_kb4 = (K + 127) / 128;
  g.C = static_cast<cb::bf16*>(C);
  g.ldc = ldc;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.sfa = static_cast<const unsigned char*>(sfa);
  g.sfb = static_cast<const unsigned char*>(sfb);
  g.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a_e5m2 && b_e5m2) return -4;   // e5m2 x e5m2 is not a training combination; keep the instantiations few
  if (a_e5m2) return cbmx::launch<1, 0>(ta, tb, g, s);
  if (b_e5m2) return cbmx::launch<0, 1>(ta, tb, g, s);
  return cbmx::launch<0, 0>(ta, tb, g, s);
}

// Rows per B tile of the CTA-pair kernel: the B scales handed to cb_mxgemm_pair must be packed for tiles of
// this many rows (cb_mxfp8_quant_packed with tile_rows = this value).
int cb_mxgemm_pair_tile_rows() { return cbmx::P_BN; }

// Bytes of the packed scale buffer when the rows are grouped in tiles of `tile_rows` (each tile padded to a
// multiple of 128 rows).
long long cb_mxgemm_sf_bytes_tiled(long long rows, int K, int tile_rows) {
  const long long tiles = (rows + tile_rows - 1) / tile_rows;
  const long long atoms_per_tile = (tile_rows + 127) / 128;
  const long long kb4 = (K + 127) / 128;
  return tiles * atoms_per_tile * kb4 * 512;
}

// The same product on CTA pairs (256 x 192 tiles).  sfa as for cb_mxgemm; sfb packed for 192-row tiles.
// C must be 16-byte aligned with a pitch that is a multiple of 8 elements (TMA-store epilogue).
int cb_mxgemm_pair(const void* Aq, const void* Bq, const void* sfa, const void* sfb, void* C, const void* bias, int M,
                   int N, int K, long long lda, long long ldb, long long ldc, int a_e5m2, int b_e5m2, int* status,
                   void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || sfa == nullptr || sfb == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(sfa) & 15) != 0 || (reinterpret_cast<uintptr_t>(sfb) & 15) != 0) return -3;
  if ((reinterpret_cast<uintptr_t>(C) & 15) != 0 || (ldc * 2) % 16 != 0) return -2;
  if (a_e5m2 && b_e5m2) return -4;
  CUtensorMap ta, tb, tc;
  int e = cbhost::make_tmap(&ta, Aq, K, M, lda, cbmx::BKB, cbmx::BM, 1);
  if (e) return e;
  e = cbhost::make_tmap(&tb, Bq, K, N, ldb, cbmx::BKB, cbmx::P_BNH, 1);
  if (e) return e;
  e = cbhost::make_tmap(&tc, C, N, M, ldc, 64, 32, 2);
  if (e) return e;
  cbmx::PairArgs g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_pairs = (M + 2 * cbmx::BM - 1) / (2 * cbmx::BM);
  g.num_n_tiles = (N + cbmx::P_BN - 1) / cbmx::P_BN;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.sf_kb4 = (K + 127) / 128;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.sfa = static_cast<const unsigned char*>(sfa);
  g.sfb = static_cast<const unsigned char*>(sfb);
  g.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a_e5m2) return cbmx::launch_pair<1, 0>(ta, tb, tc, g, s);
  if (b_e5m2) return cbmx::launch_pair<0, 1>(ta, tb, tc, g, s);
  return cbmx::launch_pair<0, 0>(ta, tb, tc, g, s);
}

}  // extern "C"
