// Two-CTA tcgen05 GEMM: C[M,N] = A[M,K] * B[N,K]^T (bf16 in / out, fp32 accumulation) with one
// 256 x BN output tile per CTA pair (`tcgen05.mma.cta_group::2`), BN = 256, 224 or 192.
//
// Why pairs: with one CTA per tile (gemm.cu, 128 x 256) every k-block of 64 needs 48 KB of operands per 512 MMA
// cycles and SM; the shared-memory ring then holds about one memory latency of data and every L2 miss reaches
// the MMA issuer.  A CTA pair shares the B tile: each CTA loads its own 128 rows of A and only HALF of the
// rows of B (32 KB per k-block and SM), the tensor cores of both SMs read the two halves from both
// shared memories, and the ring is six stages deep instead of four.
//
// Work distribution (stream-K).  A fine-tuning step multiplies a few thousand tokens by weights of a few
// thousand columns: 76 ... 1216 tiles for 74 CTA pairs, so whole tiles per pair leave up to half of the last
// round idle.  Tiles are therefore handed out in two regions: the first `sk_tiles` tiles are cut along K into
// equal runs of k-blocks, one run per pair (a pair finishes the tile its predecessor started, computes whole
// tiles, starts one for its successor); the remaining tiles, a multiple of the pair count, are computed whole.
// A partial tile is added (TMA reduce-add, fp32) into a per-tile slot of a workspace; every 32-row strip of a
// slot has an arrival counter, and the warp that arrives last reads the sum back, applies the epilogue, stores
// bf16 and leaves the strip and its counter zero for the next launch.  Nobody waits for anybody.
//
// Structure (192 threads per CTA, cluster of 2 along x):
//   warp 0      TMA producer of this CTA's A rows and B half (non-multicast loads into the CTA's own shared
//               memory; the peer CTA's loads complete on the LEADER's `full` barrier, so the MMA issuer waits
//               on one barrier per stage and no relay is needed)
//   warp 1      leader CTA (rank 0): issues the MMAs for the pair; `tcgen05.commit ... multicast::cluster`
//               releases the stage / publishes the accumulator in both CTAs
//   warps 2-5   epilogue: each CTA drains its own 128 TMEM lanes (its 128 rows of the 256-row tile) through a
//               swizzled staging buffer and TMA stores; accumulators are double buffered (2 x 256 columns).
// Every wait is bounded (common.cuh); a CTA that gives up still reaches the closing cluster barrier, and so
// does its peer once its own waits expire, so the pair always leaves together.
//
// The reference has no GEMM of its own (cuBLAS behind nn.Linear); nothing to cite.
#include <cstring>
#include "common.cuh"
#include "host_common.h"

namespace cb2 {
using namespace cb;

constexpr int BM = 128;          // rows of A (and of the accumulator) per CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = 128 * BK * 2;            // room for the widest B half (128 rows)
constexpr int STG_OFFSET = STAGES * (A_BYTES + B_BYTES);
constexpr int BAR_OFFSET = STG_OFFSET + 4 * 8192;
constexpr int SMEM_TOTAL = BAR_OFFSET + 512 + 1024;
constexpr int WS_CTR_BYTES = 16384;              // arrival counters in front of the fp32 slots of the workspace
constexpr int MAX_SK_TILES = 2 * 74 + 8;         // slots the counters are sized for (148 SMs -> 74 pairs)

struct Args {
  int M, N, K;
  int num_m_pairs, num_n_tiles, num_tiles, num_kb;
  // Second operand pair: C = A B^T + A2 B2^T.  Its k-blocks follow the num_kb1 k-blocks of the first pair in the
  // same accumulator (num_kb counts both), which is how a low-rank adapter's  (x A^T) B^T  joins the frozen
  // projection without a second pass over the output.  num_kb1 == num_kb: no second pair.
  int num_kb1;
  // stream-K region: tiles [0, sk_tiles) are cut along K; pair p owns sk_q (+1 if p < sk_r) consecutive
  // k-blocks of the region's tile-major list.  sk_tiles == 0: whole tiles only.
  int sk_tiles, sk_q, sk_r;
  float* ws;               // fp32 slots [sk_tiles][256][BN]
  unsigned int* ctr;       // arrival counters [sk_tiles][8]   (2 CTAs x 4 epilogue warps)
  void* C;                 // output (needed for accumulate and for the narrow tail columns)
  long long ldc;
  int out_fp32;
  int accumulate;
  const bf16* bias;        // [N] or null
  const bf16* addend;      // [M, N] with row pitch ld_add, or null (residual)
  long long ld_add;
  const float* row_scale;  // fp8 operands: C = (A_q B_q^T) * row_scale[m] * col_scale[n]; null for bf16 operands
  const float* col_scale;
  int* status;
  // ---- tensor-parallel fusion (TP = 1 instantiations only; same contract as cb_gemm_bf16_tp in gemm.cu)
  // all-gather -> GEMM: the rows of A arrive in panels of `panel_pairs` 256-row tiles, one panel per source rank,
  // pushed into local memory by the peers; flag[src] reaches *panel_epoch once panel src is complete
  const unsigned long long* panel_flags;
  const unsigned long long* panel_epoch;
  int panel_pairs;
  int panel_self;                 // the panel this rank produced itself (never waited for)
  int rot_pairs;                  // row tiles are visited starting here, so every rank begins with its own panel
  unsigned long long peer_wait_ns;
  // GEMM -> reduce-scatter: output rows belong to `push_rows` rows per owner rank; the epilogue stores each tile
  // through push_c[owner] (a peer mapping, pre-offset so that the global row indexes it with pitch ldc)
  unsigned long long push_c[16];
  int push_rows;
  // ---- gated-activation epilogue (GLU = 1 instantiation only): B is the fused gate | up weight [2 * glu_i, K]
  int glu_i;
};

__device__ __forceinline__ void umma_f16_ss_2cta(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the same MMA for 8-bit floating-point operands (e4m3 / e5m2 chosen by the instruction descriptor), K = 32 per MMA
__device__ __forceinline__ void umma_f8_ss_2cta(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// instruction descriptor for kind::f8f6f4: fp32 accumulator, operand formats 0 = e4m3, 1 = e5m2, both K-major
__host__ __device__ constexpr uint32_t umma_idesc_fp8(int m, int n, int a_fmt, int b_fmt) {
  return (1u << 4) | (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// TMA load issued by either CTA of a pair whose completion is counted on a barrier that may live in the peer's
// shared memory (`bar_cluster_addr` is a shared::cluster address).  No multicast: the data goes to this CTA only.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

// One pair's walk over its work: first its run of k-blocks in the stream-K region, then its whole tiles.
struct Segments {
  long long u, u_end;
  int dp_next, stride;
  __device__ __forceinline__ Segments(const Args& g, int pair, int num_pairs) {
    u = static_cast<long long>(pair) * g.sk_q + (pair < g.sk_r ? pair : g.sk_r);
    u_end = g.sk_tiles > 0 ? u + g.sk_q + (pair < g.sk_r ? 1 : 0) : u;
    if (g.sk_tiles == 0) u = u_end = 0;
    dp_next = g.sk_tiles + pair;
    stride = num_pairs;
  }
  __device__ __forceinline__ bool next(const Args& g, int& tile, int& kb0, int& kb1) {
    if (u < u_end) {
      tile = static_cast<int>(u / g.num_kb);
      kb0 = static_cast<int>(u - static_cast<long long>(tile) * g.num_kb);
      const long long left = u_end - u;
      const int rem = g.num_kb - kb0;
      kb1 = kb0 + (left < rem ? static_cast<int>(left) : rem);
      u += kb1 - kb0;
      return true;
    }
    if (dp_next < g.num_tiles) {
      tile = dp_next;
      dp_next += stride;
      kb0 = 0;
      kb1 = g.num_kb;
      return true;
    }
    return false;
  }
};
// which pair owns k-block unit `u` of the stream-K region
__device__ __forceinline__ int pair_of_unit(const Args& g, long long u) {
  const long long head = static_cast<long long>(g.sk_r) * (g.sk_q + 1);
  return u < head ? static_cast<int>(u / (g.sk_q + 1)) : g.sk_r + static_cast<int>((u - head) / g.sk_q);
}

// A_MN / B_MN: 0 = operand stored [rows, K] (K contiguous), 1 = stored [K, rows] (rows contiguous), exactly as in
// gemm.cu, so forward (0,0), dgrad (0,1) and wgrad (1,1) need no transposed copies.
// KIND: 0 = bf16 operands (kind::f16, 64 elements per k-block), 1 = e4m3 operands (kind::f8f6f4, 128 elements per
// k-block, K-major only).  Either way a k-block row is 128 bytes and one MMA consumes 32 bytes of it, so the
// shared-memory layout, the descriptors and the pipeline are identical.
// BN: columns of the pair's tile (256, 224 or 192); each CTA loads BN / 2 rows of B.
template <int BN, int A_MN, int B_MN, int KIND, int TP = 0, int GLU = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmW,
               const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, const Args g) {
  constexpr int BNH = BN / 2;
  constexpr uint32_t TMEM_COLS = 512;                                    // two accumulators, 256 columns apart
  constexpr uint32_t IDESC = KIND ? umma_idesc_fp8(2 * BM, BN, 0, 0)
                                  : umma_idesc_bf16(2 * BM, BN, A_MN, B_MN);      // M = 256 across the pair
  constexpr int BKE = KIND ? 2 * BK : BK;                                // elements per k-block
  // bytes one CTA brings in per stage: K-major B loads exactly BNH rows; MN-major B loads whole 64-column atoms
  constexpr int B_LOAD = B_MN ? ((BNH + 63) / 64) * 8192 : BNH * BK * 2;
  constexpr uint32_t STAGE_TX = 2u * (A_BYTES + B_LOAD);                 // both CTAs complete on the leader's barrier

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + BAR_OFFSET);       // (leader) the stage landed in both CTAs
  uint64_t* empty = full + STAGES;                                       // stage consumed (multicast commit)
  uint64_t* tfull = empty + STAGES;                                      // accumulator complete (multicast commit)
  uint64_t* tempty = tfull + 2;                                          // (leader) accumulator drained by both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // warp-uniform for the compiler too
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull + a, 1);
      mbar_init(tempty + a, 8);                                          // 4 epilogue warps in each CTA
    }
    mbar_fence_init();
    *abort_flag = (g.status[0] != 0) ? 1 : 0;
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  __syncthreads();
  cluster_sync_all();                                                    // barriers of both CTAs are initialised
  // Poisoned by an earlier timeout?  Both CTAs take the LEADER's view, so the pair always decides alike and
  // no cluster barrier below is ever left waiting for a CTA that went home.
  const uint32_t poisoned = ld_shared_cluster_u32(mapa_u32(smem_u32(const_cast<int*>(abort_flag)), 0));
  cluster_sync_all();                                                    // nobody leaves while its flag is being read
  if (poisoned != 0) return;
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  cluster_sync_all();                                                    // both halves of the pair hold their TMEM
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (each CTA: its A rows, its B half)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t full_leader = mapa_u32(smem_u32(full), 0);
      Segments seg(g, pair, num_pairs);
      int t, kb0, kb1;
      while (ok && seg.next(g, t, kb0, kb1)) {
        int mp = t % g.num_m_pairs;
        if (TP) {
          mp += g.rot_pairs;
          if (mp >= g.num_m_pairs) mp -= g.num_m_pairs;
        }
        const int nt = t / g.num_m_pairs;
        const int a_row = mp * 2 * BM + static_cast<int>(rank) * BM;
        // GLU: the leader's half of B holds the gate rows of activation columns [nt * BNH, +BNH), the peer's half
        // the up rows of the same columns (glu_i rows further down in the fused gate|up weight)
        const int b_row = GLU ? nt * BNH + static_cast<int>(rank) * g.glu_i : nt * BN + static_cast<int>(rank) * BNH;
        if (TP && g.panel_pairs > 0) {
          // rows of this tile come from rank `src`: wait (bounded) until its push kernel has signalled
          const int src = mp / g.panel_pairs;
          if (src != g.panel_self) {
            const unsigned long long want = *g.panel_epoch;
            const uint64_t t0 = globaltimer_ns();
            while (ld_acquire_sys_u64(g.panel_flags + src) < want) {
              if (*abort_flag) { ok = false; break; }
              if (globaltimer_ns() - t0 > g.peer_wait_ns) {
                *abort_flag = 1;
                atomicCAS(g.status, 0, CB_ERR_WAIT_PEER);
                g.status[1] = src;
                g.status[2] = blockIdx.x;
                __threadfence();
                ok = false;
                break;
              }
              __nanosleep(128);
            }
            if (!ok) break;
            fence_proxy_async_all();   // the peer's generic-proxy stores are read by TMA (async proxy) below
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          if (leader) mbar_expect_tx(full + stage, STAGE_TX);
          const uint32_t bar = full_leader + stage * 8;
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          const bool second = kb >= g.num_kb1;                 // k-blocks of the second operand pair
          const CUtensorMap* ma = second ? &tmA2 : &tmA;
          const CUtensorMap* mb = second ? &tmB2 : &tmB;
          const int kk = second ? kb - g.num_kb1 : kb;
          if (A_MN == 0) {
            tma_load_2d_pair(a_dst, ma, bar, kk * BKE, a_row);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * 8192, ma, bar, a_row + j * 64, kk * BK);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(b_dst, mb, bar, kk * BKE, b_row);
          } else {
#pragma unroll
            for (int j = 0; j < (BNH + 63) / 64; ++j) tma_load_2d_pair(b_dst + j * 8192, mb, bar, b_row + j * 64, kk * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (leader) {
      // --------------------------------------------------------- MMA issuer for the pair
      // The whole warp walks the schedule with warp-uniform control flow and one elected lane issues, so stage
      // addresses and descriptors live in uniform registers (see elect_one).
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t seg_cnt = 0;
      Segments seg(g, pair, num_pairs);
      int t, kb0, kb1;
      while (ok && seg.next(g, t, kb0, kb1)) {
        const uint32_t acc = seg_cnt & 1u;
        const uint32_t acc_phase = (seg_cnt >> 1) & 1u;
        ++seg_cnt;
        ok = __all_sync(0xffffffffu, mbar_wait(tempty + acc, acc_phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_TMEM_EMPTY));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 256;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = __all_sync(0xffffffffu, mbar_wait(full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_FULL));
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_base = smem_u32(sB + stage * B_BYTES);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t adesc = A_MN ? umma_smem_desc(a_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc(a_base + k * 32, 16, 1024);
              const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc(b_base + k * 32, 16, 1024);
              const uint32_t accum = (kb != kb0 || k != 0) ? 1u : 0u;
              if (KIND) umma_f8_ss_2cta(d_tmem, adesc, bdesc, IDESC, accum);
              else umma_f16_ss_2cta(d_tmem, adesc, bdesc, IDESC, accum);
            }
            umma_commit_2cta(empty + stage);    // frees this stage in both CTAs once the MMAs retire
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && elect_one()) umma_commit_2cta(tfull + acc);  // accumulator complete, visible to both epilogues
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (4 warps, one TMEM lane quarter each)
    const int q = warp & 3;
    const uint32_t tempty_leader = mapa_u32(smem_u32(tempty), 0);
    uint8_t* stg = smem + STG_OFFSET + (warp - 2) * 8192;
    uint32_t seg_cnt = 0;
    bool ok = true;
    int buf = 0;
    Segments seg(g, pair, num_pairs);
    int t, kb0, kb1;

    // fused math on 32 consecutive columns of this thread's row, then bf16 / fp32 packing is left to the caller
    auto fuse32 = [&](float* v, int row, bool row_ok, int col0) {
      if (KIND && g.row_scale != nullptr) {
        const float rs = row_ok ? g.row_scale[row] : 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= rs * (col0 + j < g.N ? g.col_scale[col0 + j] : 0.f);
      }
      if (g.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < g.N) v[j] += __bfloat162float(g.bias[col0 + j]);
      }
      if (g.addend != nullptr && row_ok) {
        const bf16* ap = g.addend + static_cast<long long>(row) * g.ld_add + col0;
        if (col0 + 32 <= g.N && (reinterpret_cast<uintptr_t>(ap) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 u = reinterpret_cast<const uint4*>(ap)[j];
            const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y);
            const float2 a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
            v[8 * j + 0] += a0.x; v[8 * j + 1] += a0.y; v[8 * j + 2] += a1.x; v[8 * j + 3] += a1.y;
            v[8 * j + 4] += a2.x; v[8 * j + 5] += a2.y; v[8 * j + 6] += a3.x; v[8 * j + 7] += a3.y;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < g.N) v[j] += __bfloat162float(ap[j]);
        }
      }
      if (g.accumulate && row_ok) {
        if (g.out_fp32) {
          const float* cp = reinterpret_cast<const float*>(g.C) + static_cast<long long>(row) * g.ldc + col0;
          if (col0 + 32 <= g.N && (reinterpret_cast<uintptr_t>(cp) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 o = reinterpret_cast<const float4*>(cp)[j];
              v[4 * j] += o.x; v[4 * j + 1] += o.y; v[4 * j + 2] += o.z; v[4 * j + 3] += o.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < g.N) v[j] += cp[j];
          }
        } else {
          const bf16* cp = reinterpret_cast<const bf16*>(g.C) + static_cast<long long>(row) * g.ldc + col0;
          if (col0 + 32 <= g.N && (reinterpret_cast<uintptr_t>(cp) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 u = reinterpret_cast<const uint4*>(cp)[j];
              const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y);
              const float2 a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
              v[8 * j + 0] += a0.x; v[8 * j + 1] += a0.y; v[8 * j + 2] += a1.x; v[8 * j + 3] += a1.y;
              v[8 * j + 4] += a2.x; v[8 * j + 5] += a2.y; v[8 * j + 6] += a3.x; v[8 * j + 7] += a3.y;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < g.N) v[j] += __bfloat162float(cp[j]);
          }
        }
      }
    };
    // one staging buffer -> global memory through `map` (store, or fp32 add for partial tiles)
    auto flush = [&](const CUtensorMap* map, int x, int y, bool add, bool active) {
      CB_DEBUG_CHECK_ST(g.status, !active || (x >= 0 && y >= 0 && (x * ((add || g.out_fp32) ? 4 : 2)) % 16 == 0),
                        CB_DBG_TMA_COORD, x);
      fence_async_smem();
      __syncwarp();
      if (lane == 0 && active) {
        if (add) tma_reduce_add_2d(map, stg + buf * 4096, x, y);
        else tma_store_2d(map, stg + buf * 4096, x, y);
        tma_store_commit();
      }
      buf ^= 1;
    };
    auto stage_fp32 = [&](const uint32_t* r) {
      if (lane == 0) tma_store_wait_read<1>();                // the buffer written two stores ago has been read out
      __syncwarp();
      uint8_t* dstrow = stg + buf * 4096 + lane * 128;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        const uint4 u = make_uint4(r[4 * cc], r[4 * cc + 1], r[4 * cc + 2], r[4 * cc + 3]);
        *reinterpret_cast<uint4*>(dstrow + ((cc ^ (lane & 7)) << 4)) = u;
      }
    };
    auto stage_bf16 = [&](const uint32_t* r) {                // 64 values -> 128-byte row
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
      uint8_t* dstrow = stg + buf * 4096 + lane * 128;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        uint4 u;
        u.x = pack_bf16x2(__uint_as_float(r[8 * cc + 0]), __uint_as_float(r[8 * cc + 1]));
        u.y = pack_bf16x2(__uint_as_float(r[8 * cc + 2]), __uint_as_float(r[8 * cc + 3]));
        u.z = pack_bf16x2(__uint_as_float(r[8 * cc + 4]), __uint_as_float(r[8 * cc + 5]));
        u.w = pack_bf16x2(__uint_as_float(r[8 * cc + 6]), __uint_as_float(r[8 * cc + 7]));
        *reinterpret_cast<uint4*>(dstrow + ((cc ^ (lane & 7)) << 4)) = u;
      }
    };
    // finished values of `ncol` (32 or 64) columns starting at colbase, rows row0w .. row0w + 31, to C
    auto emit = [&](uint32_t* r, int ncol, int colbase, int row0w, int row, bool row_ok) {
      fuse32(reinterpret_cast<float*>(r), row, row_ok, colbase);
      if (ncol == 64) fuse32(reinterpret_cast<float*>(r + 32), row, row_ok, colbase + 32);
      if (g.out_fp32) {
        stage_fp32(r);
        flush(&tmC, colbase, row0w, false, row0w < g.M);
      } else if (ncol == 64 && TP && g.push_rows > 0) {
        // reduce-scatter epilogue: these 32 rows live on rank row0w / push_rows; plain 16-byte stores to the peer
        // from the staged tile, 8 lanes per 128-byte row segment (full lines on the wire)
        stage_bf16(r);
        __syncwarp();
        bf16* push_base = reinterpret_cast<bf16*>(g.push_c[row0w / g.push_rows]);
        const int chunk = lane & 7;
        const int ccol = colbase + chunk * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = (lane >> 3) + 4 * i;
          const int grow = row0w + rr;
          CB_DEBUG_CHECK_ST(g.status, grow / g.push_rows == row0w / g.push_rows || grow >= g.M, CB_DBG_PUSH_ROW, grow);
          if (grow < g.M && ccol < g.N) {
            const uint4 u = *reinterpret_cast<const uint4*>(stg + buf * 4096 + rr * 128 + ((chunk ^ (rr & 7)) << 4));
            *reinterpret_cast<uint4*>(push_base + static_cast<long long>(grow) * g.ldc + ccol) = u;
          }
        }
        __syncwarp();
        buf ^= 1;
      } else if (ncol == 64) {
        stage_bf16(r);
        flush(&tmC, colbase, row0w, false, row0w < g.M);
      } else {
        // narrow tail of a tile whose width is not a multiple of 64 (BN = 224): 32 bf16 per row, plain stores
        if (row_ok) {
          bf16* cp = reinterpret_cast<bf16*>(g.C) + static_cast<long long>(row) * g.ldc + colbase;
          if (colbase + 32 <= g.N && (reinterpret_cast<uintptr_t>(cp) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              u.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              u.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              u.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              reinterpret_cast<uint4*>(cp)[j] = u;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (colbase + j < g.N) cp[j] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
    };

    while (ok && seg.next(g, t, kb0, kb1)) {
      int mp = t % g.num_m_pairs;
      if (TP) {
        mp += g.rot_pairs;
        if (mp >= g.num_m_pairs) mp -= g.num_m_pairs;
      }
      const int nt = t / g.num_m_pairs;
      const uint32_t acc = seg_cnt & 1u;
      const uint32_t acc_phase = (seg_cnt >> 1) & 1u;
      ++seg_cnt;
      bool w = mbar_wait(tfull + acc, acc_phase, abort_flag, g.status, CB_ERR_WAIT_TMEM_FULL);
      w = __all_sync(0xffffffffu, w);
      if (!w) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 256;
      const int row0w = mp * 2 * BM + static_cast<int>(rank) * BM + q * 32;
      const int row = row0w + lane;
      const bool row_ok = row < g.M;
      const bool whole = (kb0 == 0 && kb1 == g.num_kb);

      if (GLU) {
        // Accumulator columns [0, BNH) are the gate, [BNH, BN) the up projection of activation columns
        // nt * BNH ...  Per 64 columns: gate -> C (kept as bf16 pairs), up -> C, silu(gate) * up -> the activation
        // tensor (map tmW), all three through the staging buffers and TMA stores.  The product uses the values as
        // rounded to bf16 for C, i.e. what the stand-alone kernel would read back.
#pragma unroll 1
        for (int c0 = 0; c0 < BNH; c0 += 64) {
          const int acol = nt * BNH + c0;
          if (acol >= g.glu_i) break;                         // uniform across the warp
          uint32_t r[64], gp[32];
          tmem_ld_32x32(t_row + c0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_ld_32x32(t_row + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_ld_wait();
          fuse32(reinterpret_cast<float*>(r), row, row_ok, acol);
          fuse32(reinterpret_cast<float*>(r + 32), row, row_ok, acol + 32);
#pragma unroll
          for (int j = 0; j < 32; ++j) gp[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
          stage_bf16(r);
          flush(&tmC, acol, row0w, false, row0w < g.M);
          tmem_ld_32x32(t_row + BNH + c0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_ld_32x32(t_row + BNH + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_ld_wait();
          fuse32(reinterpret_cast<float*>(r), row, row_ok, g.glu_i + acol);
          fuse32(reinterpret_cast<float*>(r + 32), row, row_ok, g.glu_i + acol + 32);
          stage_bf16(r);
          flush(&tmC, g.glu_i + acol, row0w, false, row0w < g.M);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float2 gt = unpack_bf16x2(gp[j]);
            const float2 up = unpack_bf16x2(pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])));
            // silu(g) = g sigmoid(g) = h + h tanh(h) with h = g / 2: one special-function instruction and three
            // FMA-pipe instructions per element (the epilogue warps run one per scheduler, so every dependent
            // instruction costs its full latency; an exp2, a reciprocal and its refinement would not fit the tile time)
            const float h0 = 0.5f * gt.x, h1 = 0.5f * gt.y;
            r[2 * j] = __float_as_uint(fmaf(h0, tanh_approx(h0), h0) * up.x);
            r[2 * j + 1] = __float_as_uint(fmaf(h1, tanh_approx(h1), h1) * up.y);
          }
          stage_bf16(r);
          flush(&tmW, acol, row0w, false, row0w < g.M);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(tempty + acc);
          else mbar_arrive_remote(tempty_leader + acc * 8);
        }
      } else if (whole) {
        const int step = g.out_fp32 ? 32 : 64;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += step) {
          const int colbase = nt * BN + c0;
          if (colbase >= g.N) break;                          // uniform across the warp
          const int ncol = (!g.out_fp32 && c0 + 64 <= BN) ? 64 : 32;
          uint32_t r[64];
          tmem_ld_32x32(t_row + c0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          if (ncol == 64) tmem_ld_32x32(t_row + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_ld_wait();
          emit(r, ncol, colbase, row0w, row, row_ok);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(tempty + acc);
          else mbar_arrive_remote(tempty_leader + acc * 8);
        }
      } else {
        // ---- partial tile: add this run's fp32 sums into the tile's workspace slot
        const int ws_row0 = t * 256 + static_cast<int>(rank) * BM + q * 32;       // row of the [sk_tiles * 256, BN] map
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (nt * BN + c0 >= g.N) break;
          uint32_t r[32];
          tmem_ld_32x32(t_row + c0, r);
          tmem_ld_wait();
          stage_fp32(r);
          flush(&tmW, c0, ws_row0, true, true);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {                                      // the accumulator is free again
          if (leader) mbar_arrive(tempty + acc);
          else mbar_arrive_remote(tempty_leader + acc * 8);
        }
        // arrival: my adds are complete and visible before the counter moves
        unsigned int old = 0;
        if (lane == 0) {
          tma_store_wait_all();
          fence_proxy_async_all();
          __threadfence();
          const int first = pair_of_unit(g, static_cast<long long>(t) * g.num_kb);
          const int last = pair_of_unit(g, static_cast<long long>(t + 1) * g.num_kb - 1);
          unsigned int* c = g.ctr + t * 8 + static_cast<int>(rank) * 4 + q;
          old = atomicAdd(c, 1u);
          old = (old == static_cast<unsigned int>(last - first)) ? 1u : 0u;       // last - first + 1 contributors
          if (old) {
            __threadfence();
            *c = 0u;                                          // counter ready for the next launch
          }
        }
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old) {
          // ---- last arrival for this 32-row strip: read the sum, clear the slot, run the epilogue
          float* wrow = g.ws + (static_cast<long long>(t) * 256 + static_cast<int>(rank) * BM + q * 32 + lane) * BN;
          const int step = g.out_fp32 ? 32 : 64;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += step) {
            const int colbase = nt * BN + c0;
            if (colbase >= g.N) break;
            const int ncol = (!g.out_fp32 && c0 + 64 <= BN) ? 64 : 32;
            uint32_t r[64];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (4 * j < ncol) {
                const float4 x = __ldcg(reinterpret_cast<const float4*>(wrow + c0) + j);
                r[4 * j] = __float_as_uint(x.x); r[4 * j + 1] = __float_as_uint(x.y);
                r[4 * j + 2] = __float_as_uint(x.z); r[4 * j + 3] = __float_as_uint(x.w);
                __stcg(reinterpret_cast<float4*>(wrow + c0) + j, make_float4(0.f, 0.f, 0.f, 0.f));
              }
            }
            emit(r, ncol, colbase, row0w, row, row_ok);
          }
          // columns beyond N inside the slot were added to as well: clear them too
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            if (nt * BN + c0 < g.N) continue;
#pragma unroll
            for (int j = 0; j < 8; ++j) __stcg(reinterpret_cast<float4*>(wrow + c0) + j, make_float4(0.f, 0.f, 0.f, 0.f));
          }
        }
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

}  // namespace cb2

namespace {

// per-device workspace handed in by the host framework (cb_gemm2sm_set_workspace); absent: whole tiles only
constexpr int MAX_DEVICES = 64;
void* g_ws_ptr[MAX_DEVICES] = {};
unsigned long long g_ws_bytes[MAX_DEVICES] = {};

template <int BN, int A_MN, int B_MN, int KIND = 0, int TP = 0, int GLU = 0>
int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tw, const cb2::Args& g,
            int pairs, cudaStream_t s, const CUtensorMap* ta2 = nullptr, const CUtensorMap* tb2 = nullptr) {
  auto kern = cb2::gemm2sm_kernel<BN, A_MN, B_MN, KIND, TP, GLU>;
  static bool configured = false;
  if (!configured) {
    CB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cb2::SMEM_TOTAL));
    configured = true;
  }
  kern<<<2 * pairs, cb2::THREADS, cb2::SMEM_TOTAL, s>>>(ta, tb, tc, tw, ta2 ? *ta2 : ta, tb2 ? *tb2 : tb, g);
  return static_cast<int>(cudaGetLastError());
}

template <int BN>
int dispatch_layout(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                    const CUtensorMap& tw, const cb2::Args& g, int pairs, cudaStream_t s,
                    const CUtensorMap* ta2 = nullptr, const CUtensorMap* tb2 = nullptr) {
  if (!a_mn && !b_mn) return launch2<BN, 0, 0>(ta, tb, tc, tw, g, pairs, s, ta2, tb2);
  if (!a_mn && b_mn) return launch2<BN, 0, 1>(ta, tb, tc, tw, g, pairs, s, ta2, tb2);
  if (a_mn && b_mn) return launch2<BN, 1, 1>(ta, tb, tc, tw, g, pairs, s, ta2, tb2);
  return launch2<BN, 1, 0>(ta, tb, tc, tw, g, pairs, s, ta2, tb2);
}

// Whole tiles take ceil(T / pairs) rounds; cut along K the work takes T / pairs rounds plus the fixups (partial
// sums through L2, the last arrival's read-back and a burst of them when every pair ends on a partial tile),
// measured at about 36 us, i.e. 72 / num_kb rounds of a 64-wide k-block at ~0.5 us.  Worth it for long K and a
// mostly empty last round (weight gradients over thousands of tokens), not for the K = 896 projections.
bool stream_k_pays(long long T, int pairs, int num_kb) {
  if (pairs < 2 || T % pairs == 0) return false;
  const double whole = static_cast<double>((T + pairs - 1) / pairs);
  const double split = static_cast<double>(T) / pairs + 72.0 / num_kb;
  return split < whole - 0.05;
}

// tile width with the least padding of N (ties: the widest)
int pick_bn(int N) {
  int best = 256;
  long long best_pad = -1;
  for (int bn : {256, 224, 192}) {
    const long long pad = static_cast<long long>((N + bn - 1) / bn) * bn - N;
    if (best_pad < 0 || pad < best_pad) {
      best_pad = pad;
      best = bn;
    }
  }
  return best;
}

// Fills the stream-K fields of `g` for `pairs` resident pairs.  Returns the number of tile slots the workspace
// needs (0: whole tiles only).
int plan_stream_k(cb2::Args* g, int pairs, int bn, int device, int allow) {
  g->sk_tiles = 0;
  g->sk_q = g->sk_r = 0;
  g->ws = nullptr;
  g->ctr = nullptr;
  const int T = g->num_tiles;
  if (!allow || pairs < 2 || T % pairs == 0 || device < 0 || device >= MAX_DEVICES || g_ws_ptr[device] == nullptr) return 0;
  const int full = T / pairs, rem = T % pairs;
  if (allow != 2 && !stream_k_pays(T, pairs, g->num_kb)) return 0;
  int sk = full >= 1 ? rem + pairs : T;                      // every pair gets between one and two tiles' worth
  if (sk > T) sk = T;
  if (sk > cb2::MAX_SK_TILES) return 0;
  const long long units = static_cast<long long>(sk) * g->num_kb;
  if (units < 4LL * pairs) return 0;                         // runs shorter than 4 k-blocks are not worth a fixup
  const unsigned long long need = cb2::WS_CTR_BYTES + static_cast<unsigned long long>(sk) * 256ull * bn * 4ull;
  if (need > g_ws_bytes[device]) return 0;
  g->sk_tiles = sk;
  g->sk_q = static_cast<int>(units / pairs);
  g->sk_r = static_cast<int>(units % pairs);
  g->ctr = static_cast<unsigned int*>(g_ws_ptr[device]);
  g->ws = reinterpret_cast<float*>(static_cast<unsigned char*>(g_ws_ptr[device]) + cb2::WS_CTR_BYTES);
  return sk;
}

}  // namespace

extern "C" {

// Whether cb_gemm2sm_bf16 can take this problem (TMA-store epilogue needs an aligned C and pitch).
int cb_gemm2sm_supported(const void* C, long long ldc, int out_fp32) {
  const int eb = out_fp32 ? 4 : 2;
  return ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * eb) % 16 == 0) ? 1 : 0;
}

// Bytes of workspace that cover every stream-K plan (arrival counters + the largest set of fp32 tile slots).
unsigned long long cb_gemm2sm_workspace_bytes() {
  return cb2::WS_CTR_BYTES + static_cast<unsigned long long>(cb2::MAX_SK_TILES) * 256ull * 256ull * 4ull;
}

// Registers a zero-filled device buffer of at least cb_gemm2sm_workspace_bytes() bytes for `device`.  The kernels
// leave it zero-filled after every launch; launches that use it must be ordered on one stream (or by events).
// ptr == null unregisters it (whole tiles only).
int cb_gemm2sm_set_workspace(int device, void* ptr, unsigned long long bytes) {
  if (device < 0 || device >= MAX_DEVICES) return -1;
  if (ptr != nullptr && ((reinterpret_cast<uintptr_t>(ptr) & 1023) != 0 || bytes < cb_gemm2sm_workspace_bytes())) return -2;
  g_ws_ptr[device] = ptr;
  g_ws_bytes[device] = ptr ? bytes : 0;
  return 0;
}

// What the dispatcher needs to know about a problem: rounds of tile time the pair kernel takes (x 1000).
int cb_gemm2sm_cost_milli(int M, int N, int K, int pairs_avail) {
  const int bn = pick_bn(N);
  const long long T = static_cast<long long>((M + 255) / 256) * ((N + bn - 1) / bn);
  const int pairs = T < pairs_avail ? static_cast<int>(T) : pairs_avail;
  int dev = 0;
  cudaGetDevice(&dev);
  const bool ws = dev >= 0 && dev < MAX_DEVICES && g_ws_ptr[dev] != nullptr;
  const long long kb = (K + 63) / 64;
  double rounds = static_cast<double>((T + pairs - 1) / pairs);
  if (ws && T * kb >= 4LL * pairs && stream_k_pays(T, pairs, static_cast<int>(kb)))
    rounds = static_cast<double>(T) / pairs + 72.0 / kb;
  return static_cast<int>(rounds * 1000.0 * bn / 256.0);
}

// C[M,N] = op(A) * op(B)^T (+bias) (+addend) (+C) on CTA pairs.  Same conventions as cb_gemm_bf16 (gemm.cu):
// a_mn / b_mn = 0 for operands stored [rows, K], 1 for [K, rows]; pitches in elements.
// flags: bit 0 = never split tiles along K, bit 1 = split whenever the last round is partial (default: only when
// it pays), bits 8.. = forced tile width (256, 224, 192; 0 = choose).
int cb_gemm2sm_bf16_ex(const void* A, const void* B, void* C, const void* bias, const void* addend, int M, int N, int K,
                       long long lda, long long ldb, long long ldc, long long ld_add, int a_mn, int b_mn, int out_fp32,
                       int accumulate, int flags, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (!cb_gemm2sm_supported(C, ldc, out_fp32)) return -2;
  int bn = flags >> 8;
  if (bn != 256 && bn != 224 && bn != 192) bn = pick_bn(N);
  if (b_mn && (ldb * 2) % 16 != 0) return -3;
  CUtensorMap ta, tb, tc, tw;
  int e;
  if (!a_mn) e = cbhost::make_tmap(&ta, A, K, M, lda, 64, cb2::BM);
  else e = cbhost::make_tmap(&ta, A, M, K, lda, 64, 64);
  if (e) return e;
  if (!b_mn) e = cbhost::make_tmap(&tb, B, K, N, ldb, 64, bn / 2);
  else e = cbhost::make_tmap(&tb, B, N, K, ldb, 64, 64);
  if (e) return e;
  e = cbhost::make_tmap(&tc, C, N, M, ldc, out_fp32 ? 32 : 64, 32, out_fp32 ? 4 : 2);
  if (e) return e;
  cb2::Args g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_pairs = (M + 2 * cb2::BM - 1) / (2 * cb2::BM);
  g.num_n_tiles = (N + bn - 1) / bn;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.num_kb = (K + cb2::BK - 1) / cb2::BK;
  g.num_kb1 = g.num_kb;
  g.C = C; g.ldc = ldc; g.out_fp32 = out_fp32; g.accumulate = accumulate;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.addend = static_cast<const cb::bf16*>(addend);
  g.ld_add = ld_add;
  g.status = status;
  int pairs = cbhost::num_sms() / 2;
  if (pairs > g.num_tiles) pairs = g.num_tiles;
  int dev = 0;
  cudaGetDevice(&dev);
  const int slots = plan_stream_k(&g, pairs, bn, dev, (flags & 1) ? 0 : ((flags & 2) ? 2 : 1));
  memset(&tw, 0, sizeof(tw));
  if (slots > 0) {
    e = cbhost::make_tmap(&tw, g.ws, bn, static_cast<unsigned long long>(slots) * 256ull, bn, 32, 32, 4);
    if (e) return e;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 256) return dispatch_layout<256>(a_mn, b_mn, ta, tb, tc, tw, g, pairs, s);
  if (bn == 224) return dispatch_layout<224>(a_mn, b_mn, ta, tb, tc, tw, g, pairs, s);
  return dispatch_layout<192>(a_mn, b_mn, ta, tb, tc, tw, g, pairs, s);
}

// Gate | up projection with the gated activation in the epilogue:
//   GU[M, 2I] = A[M, K] W[2I, K]^T (+ bias[2I]),   ACT[M, I] = silu(GU[:, :I]) * GU[:, I:]
// W holds the gate rows first, then the up rows (the fused weight as stored); both outputs are bf16.  A pair's
// tile covers 256 rows and 128 activation columns: the leader loads the 128 gate rows of those columns, its peer the
// 128 up rows, so every CTA finds gate and up of its 128 rows side by side in the accumulator.  I must be a
// multiple of 128 (returns -5 otherwise; the caller then runs the projection and the activation separately).
int cb_gemm2sm_bf16_glu(const void* A, const void* W, void* GU, void* ACT, const void* bias, int M, int I, int K,
                        long long lda, long long ldw, long long ld_gu, long long ld_act, int* status, void* stream) {
  if (M <= 0 || I <= 0 || K <= 0) return -1;
  if (I % 128 != 0) return -5;
  if (!cb_gemm2sm_supported(GU, ld_gu, 0) || !cb_gemm2sm_supported(ACT, ld_act, 0)) return -2;
  CUtensorMap ta, tb, tc, tact;
  int e = cbhost::make_tmap(&ta, A, K, M, lda, 64, cb2::BM);
  if (e) return e;
  e = cbhost::make_tmap(&tb, W, K, 2ull * I, ldw, 64, 128);
  if (e) return e;
  e = cbhost::make_tmap(&tc, GU, 2ull * I, M, ld_gu, 64, 32, 2);
  if (e) return e;
  e = cbhost::make_tmap(&tact, ACT, I, M, ld_act, 64, 32, 2);
  if (e) return e;
  cb2::Args g = {};
  g.M = M; g.N = 2 * I; g.K = K;
  g.glu_i = I;
  g.num_m_pairs = (M + 2 * cb2::BM - 1) / (2 * cb2::BM);
  g.num_n_tiles = I / 128;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.num_kb = (K + cb2::BK - 1) / cb2::BK;
  g.num_kb1 = g.num_kb;
  g.C = GU; g.ldc = ld_gu;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.status = status;
  int pairs = cbhost::num_sms() / 2;
  if (pairs > g.num_tiles) pairs = g.num_tiles;
  return launch2<256, 0, 0, 0, 0, 1>(ta, tb, tc, tact, g, pairs, static_cast<cudaStream_t>(stream));
}

// C[M,N] = A B^T + A2 B2^T (+bias) (+addend): the second product (inner dimension K2, small) is accumulated in the
// same tiles after the first (a low-rank adapter joining its frozen projection).  A / A2 are stored [M, K] / [M, K2];
// B / B2 share one layout: b_mn = 0 for [N, K] / [N, K2], 1 for [K, N] / [K2, N].  bf16 output.
int cb_gemm2sm_bf16_dual(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* bias,
                         const void* addend, int M, int N, int K, int K2, long long lda, long long ldb, long long lda2,
                         long long ldb2, long long ldc, long long ld_add, int b_mn, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K2 <= 0) return -1;
  if (!cb_gemm2sm_supported(C, ldc, 0)) return -2;
  const int bn = pick_bn(N);
  if (b_mn && ((ldb * 2) % 16 != 0 || (ldb2 * 2) % 16 != 0)) return -3;
  CUtensorMap ta, tb, ta2, tb2, tc, tw;
  int e = cbhost::make_tmap(&ta, A, K, M, lda, 64, cb2::BM);
  if (e) return e;
  e = cbhost::make_tmap(&ta2, A2, K2, M, lda2, 64, cb2::BM);
  if (e) return e;
  if (!b_mn) {
    e = cbhost::make_tmap(&tb, B, K, N, ldb, 64, bn / 2);
    if (e) return e;
    e = cbhost::make_tmap(&tb2, B2, K2, N, ldb2, 64, bn / 2);
  } else {
    e = cbhost::make_tmap(&tb, B, N, K, ldb, 64, 64);
    if (e) return e;
    e = cbhost::make_tmap(&tb2, B2, N, K2, ldb2, 64, 64);
  }
  if (e) return e;
  e = cbhost::make_tmap(&tc, C, N, M, ldc, 64, 32, 2);
  if (e) return e;
  memset(&tw, 0, sizeof(tw));
  cb2::Args g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_pairs = (M + 2 * cb2::BM - 1) / (2 * cb2::BM);
  g.num_n_tiles = (N + bn - 1) / bn;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.num_kb1 = (K + cb2::BK - 1) / cb2::BK;
  g.num_kb = g.num_kb1 + (K2 + cb2::BK - 1) / cb2::BK;
  g.C = C; g.ldc = ldc;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.addend = static_cast<const cb::bf16*>(addend);
  g.ld_add = ld_add;
  g.status = status;
  int pairs = cbhost::num_sms() / 2;
  if (pairs > g.num_tiles) pairs = g.num_tiles;
  int dev = 0;
  cudaGetDevice(&dev);
  const int slots = plan_stream_k(&g, pairs, bn, dev, 1);
  if (slots > 0) {
    e = cbhost::make_tmap(&tw, g.ws, bn, static_cast<unsigned long long>(slots) * 256ull, bn, 32, 32, 4);
    if (e) return e;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 256) return dispatch_layout<256>(0, b_mn, ta, tb, tc, tw, g, pairs, s, &ta2, &tb2);
  if (bn == 224) return dispatch_layout<224>(0, b_mn, ta, tb, tc, tw, g, pairs, s, &ta2, &tb2);
  return dispatch_layout<192>(0, b_mn, ta, tb, tc, tw, g, pairs, s, &ta2, &tb2);
}

int cb_gemm2sm_bf16(const void* A, const void* B, void* C, const void* bias, const void* addend, int M, int N, int K,
                    long long lda, long long ldb, long long ldc, long long ld_add, int a_mn, int b_mn, int out_fp32,
                    int accumulate, int* status, void* stream) {
  return cb_gemm2sm_bf16_ex(A, B, C, bias, addend, M, N, K, lda, ldb, ldc, ld_add, a_mn, b_mn, out_fp32, accumulate, 0,
                            status, stream);
}

// Tensor-parallel variants on CTA pairs (bf16 output, A stored [M, K]; same contract as cb_gemm_bf16_tp in gemm.cu):
//  * panel_rows > 0 (all-gather -> GEMM): A's rows arrive in W panels of panel_rows rows pushed by the peers;
//    panel_flags[src] (local, u64) reaches *panel_epoch when panel src is complete.  The kernel starts with this
//    rank's own panel and waits (bounded by wait_ns) per panel while the others are still in flight.
//  * push_rows > 0 (GEMM -> reduce-scatter): output rows [o * push_rows, (o + 1) * push_rows) are stored through
//    push_ptrs[o] (peer mappings, pre-offset so that the global row number indexes them with pitch ldc).
// panel_rows must be a multiple of 256 and push_rows of 32; N a multiple of 64 with push.  Returns -5 when the
// shape does not fit these tiles (the caller then uses the single-CTA kernel).
int cb_gemm2sm_bf16_tp(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                       long long ldb, long long ldc, int b_mn, const unsigned long long* panel_flags,
                       const unsigned long long* panel_epoch, int panel_rows, const unsigned long long* push_ptrs,
                       int push_rows, int W, int my_rank, unsigned long long wait_ns, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || W < 1 || W > 16 || my_rank < 0 || my_rank >= W) return -1;
  if (panel_rows < 0 || push_rows < 0 || panel_rows % 256 != 0 || push_rows % 32 != 0) return -5;
  if (panel_rows > 0 && (panel_flags == nullptr || panel_epoch == nullptr || static_cast<long long>(panel_rows) * W < M)) return -3;
  if (push_rows > 0 && (push_ptrs == nullptr || static_cast<long long>(push_rows) * W < M || N % 64 != 0 || ldc % 8 != 0)) return -5;
  if (push_rows == 0 && !cb_gemm2sm_supported(C, ldc, 0)) return -5;
  if (b_mn && (ldb * 2) % 16 != 0) return -5;
  CUtensorMap ta, tb, tc, tw;
  int e = cbhost::make_tmap(&ta, A, K, M, lda, 64, cb2::BM);
  if (e) return e;
  if (!b_mn) e = cbhost::make_tmap(&tb, B, K, N, ldb, 64, 128);
  else e = cbhost::make_tmap(&tb, B, N, K, ldb, 64, 64);
  if (e) return e;
  memset(&tc, 0, sizeof(tc));
  memset(&tw, 0, sizeof(tw));
  if (push_rows == 0) {
    e = cbhost::make_tmap(&tc, C, N, M, ldc, 64, 32, 2);
    if (e) return e;
  }
  cb2::Args g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_pairs = (M + 2 * cb2::BM - 1) / (2 * cb2::BM);
  g.num_n_tiles = (N + 255) / 256;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.num_kb = (K + cb2::BK - 1) / cb2::BK;
  g.num_kb1 = g.num_kb;
  g.C = C; g.ldc = ldc;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.status = status;
  g.peer_wait_ns = wait_ns;
  if (panel_rows > 0) {
    g.panel_flags = panel_flags;
    g.panel_epoch = panel_epoch;
    g.panel_pairs = panel_rows / 256;
    g.panel_self = my_rank;
    g.rot_pairs = (my_rank * g.panel_pairs) % g.num_m_pairs;
  }
  if (push_rows > 0) {
    g.push_rows = push_rows;
    for (int i = 0; i < W; ++i) g.push_c[i] = push_ptrs[i];
    g.rot_pairs = static_cast<int>((static_cast<long long>(my_rank) * push_rows / 256) % g.num_m_pairs);
    g.C = nullptr;
  }
  int pairs = cbhost::num_sms() / 2;
  if (pairs > g.num_tiles) pairs = g.num_tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!b_mn) return launch2<256, 0, 0, 0, 1>(ta, tb, tc, tw, g, pairs, s);
  return launch2<256, 0, 1, 0, 1>(ta, tb, tc, tw, g, pairs, s);
}

// FP8 (e4m3) GEMM on the tensor cores: C[M,N] (bf16) = (Aq[M,K] * Bq[N,K]^T) * row_scale[m] * col_scale[n] (+bias).
// Aq / Bq hold e4m3 bytes with K contiguous; pitches in bytes, multiples of 16; K a multiple of 16.
int cb_gemm2sm_fp8(const void* Aq, const void* Bq, void* C, const float* row_scale, const float* col_scale,
                   const void* bias, int M, int N, int K, long long lda, long long ldb, long long ldc, int* status,
                   void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 16 != 0 || row_scale == nullptr || col_scale == nullptr) return -1;
  if (!cb_gemm2sm_supported(C, ldc, 0)) return -2;
  CUtensorMap ta, tb, tc, tw;
  int e = cbhost::make_tmap(&ta, Aq, K, M, lda, 128, cb2::BM, 1);
  if (e) return e;
  e = cbhost::make_tmap(&tb, Bq, K, N, ldb, 128, 128, 1);
  if (e) return e;
  e = cbhost::make_tmap(&tc, C, N, M, ldc, 64, 32, 2);
  if (e) return e;
  memset(&tw, 0, sizeof(tw));
  cb2::Args g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_pairs = (M + 2 * cb2::BM - 1) / (2 * cb2::BM);
  g.num_n_tiles = (N + 255) / 256;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.num_kb = (K + 2 * cb2::BK - 1) / (2 * cb2::BK);
  g.num_kb1 = g.num_kb;
  g.C = C; g.ldc = ldc;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.row_scale = row_scale;
  g.col_scale = col_scale;
  g.status = status;
  int pairs = cbhost::num_sms() / 2;
  if (pairs > g.num_tiles) pairs = g.num_tiles;
  return launch2<256, 0, 0, 1>(ta, tb, tc, tw, g, pairs, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
