// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// TMEM, operands staged by TMA), persistent and warp-specialised:
//
//   warp 0 (one lane)  : TMA producer   global -> 128B-swizzled smem ring
//   warp 1 (one lane)  : MMA issuer     tcgen05.mma into one of two TMEM accumulators
//   warps 2..5         : epilogue       tcgen05.ld -> registers -> fused math -> global
//
// C[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation.  Each operand may be
// K-major (row = M/N index, K contiguous) or MN-major (row = K index, M/N
// contiguous), which covers forward (K,K), dgrad (K,MN) and wgrad (MN,MN)
// without transposing anything in memory.
//
// Epilogues:
//   EPI_STORE   : C = acc (+bias[n]) (+addend[m,n]) (+C), bf16 or fp32 out
//   EPI_LSE     : cut-cross-entropy forward - running (max, sum-exp) per row over
//                 a range of vocab tiles, the target logit, optional sum of logits;
//                 the logits never leave the SM
//   EPI_DLOGITS : cut-cross-entropy backward - recomputed logits turned into
//                 d(loss)/d(logits) in registers and written as bf16 for the two
//                 gradient GEMMs
//
// This replaces the cuBLAS calls behind every nn.Linear of the reference's
// training step and the fp32 cuBLAS chunk GEMMs of its cut-cross-entropy
// (reference: chronicals/kernels/cut_cross_entropy.py:915-981).
#include "common.cuh"
#include "host_common.h"

#include <string.h>

namespace cb {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

enum : int { EPI_STORE = 0, EPI_LSE = 1, EPI_DLOGITS = 2 };

struct GemmArgs {
  int M, N, K;
  int num_m_blocks, num_n_tiles, tiles_per_item, num_items;
  // EPI_STORE / EPI_DLOGITS output
  void* C;
  long long ldc;
  int out_fp32;
  int accumulate;
  const bf16* bias;
  const bf16* addend;
  long long ld_add;
  // cut-cross-entropy
  const long long* labels;  // [M], global vocab ids, ignore_index allowed
  float* part_m;            // [n_splits, M]
  float* part_s;            // [n_splits, M]
  float* part_sum;          // [n_splits, M] or null (only for label smoothing)
  float* tgt;               // [M] target logit (zero-initialised by the host)
  const float* lse;         // [M]
  const float* gscale;      // [M]  valid / n_valid
  const float* gout;        // [1]  upstream gradient of the scalar loss
  float z_weight;
  float smoothing;
  int tma_store;   // 1: the epilogue stages tiles in shared memory and writes them with TMA stores
  int V_total;     // vocabulary size for the smoothing term
  int col_offset;  // global vocab id of column 0 of B (vocab chunk or tensor-parallel shard)
  int* status;
  // ---- tensor-parallel fusion (all zero for ordinary GEMMs)
  // all-gather -> GEMM: the rows of A arrive in panels of `panel_blocks` m-blocks, one panel per source
  // rank, pushed into local memory by the peers; flag[src] reaches *panel_epoch once panel src is complete.
  const unsigned long long* panel_flags;
  const unsigned long long* panel_epoch;
  int panel_blocks;
  int panel_self;                 // the panel this rank produced itself (never waited for)
  int rot_blocks;                 // m-blocks are visited starting here, so every rank begins with its own panel
  unsigned long long peer_wait_ns;
  // GEMM -> reduce-scatter: the output rows belong to `push_blocks` m-blocks per owner rank; the epilogue
  // stores each tile through push_c[owner] (a peer mapping, pre-offset so that the global row indexes it)
  unsigned long long push_c[16];
  int push_blocks;
  // ---- split-K (skinny outputs with a long K): items beyond items_per_ksplit repeat the tiles for the next
  // K range; partial tiles are added into a zero-initialised fp32 C with red.global.add
  int items_per_ksplit;           // 0: no split
  int kb_per_split;
};

template <int BLOCK_N, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STG_OFFSET = STAGES * (A_BYTES + B_BYTES);   // epilogue staging: 4 warps x 2 x 4 KB
  static constexpr int BAR_OFFSET = STG_OFFSET + 4 * 8192;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

template <int BLOCK_N, int A_MN, int B_MN, int STAGES, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmArgs g) {
  using L = SmemLayout<BLOCK_N, STAGES>;
  constexpr int A_BYTES = L::A_BYTES, B_BYTES = L::B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_N;  // two accumulators; 256 or 512 (powers of two)
  constexpr uint32_t IDESC = umma_idesc_bf16(BLOCK_M, BLOCK_N, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // warp-uniform for the compiler too
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
  const int num_kb = (g.K + BLOCK_K - 1) / BLOCK_K;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item0 = blockIdx.x; item0 < g.num_items && ok; item0 += gridDim.x) {
        const int ks = g.items_per_ksplit > 0 ? item0 / g.items_per_ksplit : 0;
        const int item = item0 - ks * g.items_per_ksplit;
        const int kb0 = g.items_per_ksplit > 0 ? ks * g.kb_per_split : 0;
        const int kb1 = g.items_per_ksplit > 0 ? min(num_kb, kb0 + g.kb_per_split) : num_kb;
        int m_blk = item % g.num_m_blocks + g.rot_blocks;
        if (m_blk >= g.num_m_blocks) m_blk -= g.num_m_blocks;
        const int split = item / g.num_m_blocks;
        const int nt0 = split * g.tiles_per_item;
        const int nt1 = min(nt0 + g.tiles_per_item, g.num_n_tiles);
        if (g.panel_blocks > 0) {
          // rows of this m-block come from rank `src`: wait (bounded) until its push kernel has signalled
          const int src = m_blk / g.panel_blocks;
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
        for (int nt = nt0; nt < nt1 && ok; ++nt) {
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(empty + stage, phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_EMPTY)) {
              ok = false;
              break;
            }
            mbar_expect_tx(full + stage, A_BYTES + B_BYTES);
            uint8_t* a_dst = sA + stage * A_BYTES;
            uint8_t* b_dst = sB + stage * B_BYTES;
            if (A_MN == 0) {
              tma_load_2d(a_dst, &tmA, full + stage, kb * BLOCK_K, m_blk * BLOCK_M);
            } else {
#pragma unroll
              for (int j = 0; j < BLOCK_M / 64; ++j)
                tma_load_2d(a_dst + j * 8192, &tmA, full + stage, m_blk * BLOCK_M + j * 64, kb * BLOCK_K);
            }
            if (B_MN == 0) {
              tma_load_2d(b_dst, &tmB, full + stage, kb * BLOCK_K, nt * BLOCK_N);
            } else {
#pragma unroll
              for (int j = 0; j < BLOCK_N / 64; ++j)
                tma_load_2d(b_dst + j * 8192, &tmB, full + stage, nt * BLOCK_N + j * 64, kb * BLOCK_K);
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    // The whole warp walks the schedule with warp-uniform control flow and one elected lane issues, so stage
    // addresses and descriptors live in uniform registers (see elect_one).
    {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tile_cnt = 0;
      bool ok = true;
      for (int item0 = blockIdx.x; item0 < g.num_items && ok; item0 += gridDim.x) {
        const int ks = g.items_per_ksplit > 0 ? item0 / g.items_per_ksplit : 0;
        const int item = item0 - ks * g.items_per_ksplit;
        const int kb0 = g.items_per_ksplit > 0 ? ks * g.kb_per_split : 0;
        const int kb1 = g.items_per_ksplit > 0 ? min(num_kb, kb0 + g.kb_per_split) : num_kb;
        const int split = item / g.num_m_blocks;
        const int nt0 = split * g.tiles_per_item;
        const int nt1 = min(nt0 + g.tiles_per_item, g.num_n_tiles);
        for (int nt = nt0; nt < nt1 && ok; ++nt, ++tile_cnt) {
          const uint32_t acc = tile_cnt & 1u;
          const uint32_t acc_phase = (tile_cnt >> 1) & 1u;
          ok = __all_sync(0xffffffffu, mbar_wait(tempty + acc, acc_phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_TMEM_EMPTY));
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
          for (int kb = kb0; kb < kb1; ++kb) {
            ok = __all_sync(0xffffffffu, mbar_wait(full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_FULL));
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_base = smem_u32(sA + stage * A_BYTES);
            const uint32_t b_base = smem_u32(sB + stage * B_BYTES);
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                const uint64_t adesc = A_MN ? umma_smem_desc(a_base + k * 2048, 8192, 1024)
                                            : umma_smem_desc(a_base + k * 32, 16, 1024);
                const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + k * 2048, 8192, 1024)
                                            : umma_smem_desc(b_base + k * 32, 16, 1024);
                umma_f16_ss(d_tmem, adesc, bdesc, IDESC, (kb != kb0 || k != 0) ? 1u : 0u);
              }
              umma_commit(empty + stage);  // frees the smem stage once these MMAs retire
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok && elect_one()) umma_commit(tfull + acc);  // accumulator complete
        }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (4 warps, one TMEM lane quarter each)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    uint32_t tile_cnt = 0;
    bool ok = true;
    for (int item0 = blockIdx.x; item0 < g.num_items && ok; item0 += gridDim.x) {
      const int item = g.items_per_ksplit > 0 ? item0 % g.items_per_ksplit : item0;
      int m_blk = item % g.num_m_blocks + g.rot_blocks;
      if (m_blk >= g.num_m_blocks) m_blk -= g.num_m_blocks;
      const int split = item / g.num_m_blocks;
      const int nt0 = split * g.tiles_per_item;
      const int nt1 = min(nt0 + g.tiles_per_item, g.num_n_tiles);
      const int row = m_blk * BLOCK_M + row_in_tile;
      // reduce-scatter epilogue: this m-block's rows live on rank m_blk / push_blocks
      bf16* push_base = g.push_blocks > 0 ? reinterpret_cast<bf16*>(g.push_c[m_blk / g.push_blocks]) : nullptr;
      const bool row_ok = row < g.M;

      // per-row state of the cut-cross-entropy epilogues
      float run_m = -INFINITY, run_s = 0.f, run_sum = 0.f;
      int lab = -1;
      float lse_r = 0.f, gs = 0.f, coef = 1.f;
      if (EPI != EPI_STORE && row_ok) {
        const long long l = g.labels[row];
        const long long rel = l - g.col_offset;
        lab = (l >= 0 && rel >= 0 && rel < g.N) ? static_cast<int>(rel) : -1;
        if (EPI == EPI_DLOGITS) {
          lse_r = g.lse[row];
          gs = g.gscale[row] * g.gout[0];
          coef = 1.f + 2.f * g.z_weight * lse_r;
        }
      }

      for (int nt = nt0; nt < nt1 && ok; ++nt, ++tile_cnt) {
        const uint32_t acc = tile_cnt & 1u;
        const uint32_t acc_phase = (tile_cnt >> 1) & 1u;
        bool w = mbar_wait(tfull + acc, acc_phase, abort_flag, g.status, CB_ERR_WAIT_TMEM_FULL);
        w = __all_sync(0xffffffffu, w);
        if (!w) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BLOCK_N;

        if (EPI != EPI_LSE && g.tma_store) {
          // ---- staged epilogue: TMEM -> registers -> fused math -> swizzled smem tile -> TMA store.
          // Each warp owns 32 rows and two 4 KB staging buffers ([32 rows x 128 B], 16-byte chunks
          // XOR-swizzled by row & 7 to match the tensor map); stores of one buffer overlap the
          // math of the next.  Rows >= M and columns >= N are clipped by the TMA store itself.
          uint8_t* stg = smem + L::STG_OFFSET + (warp - 2) * 8192;
          const int row0w = m_blk * BLOCK_M + q * 32;
          const int cols_per_store = g.out_fp32 ? 32 : 64;
          int buf = 0;
#pragma unroll 1
          for (int c0 = 0; c0 < BLOCK_N; c0 += cols_per_store) {
            const int colbase = nt * BLOCK_N + c0;
            if (colbase >= g.N) break;  // uniform across the warp
            uint32_t r[64];
            tmem_ld_32x32(t_row + c0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            if (!g.out_fp32) tmem_ld_32x32(t_row + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
            tmem_ld_wait();
            const int nhalf = g.out_fp32 ? 1 : 2;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              if (hh >= nhalf) break;
              const int col0 = colbase + hh * 32;
              float* v = reinterpret_cast<float*>(&r[hh * 32]);
              if (EPI == EPI_DLOGITS) {
                const float sm = g.smoothing / static_cast<float>(g.V_total);
                const float l2 = lse_r * 1.4426950408889634f;
                const int rel = lab - col0;
                // (softmax * coef - sm) * gs as  fma, ex2, fma  per element; the label's -(1 - smoothing) * gs is
                // added afterwards by the few lanes whose label falls into these 32 columns (the epilogue warps
                // run one per scheduler, so every instruction in this loop is paid at its full latency)
                const float cg = coef * gs, smg = sm * gs;
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = fmaf(ex2_approx(fmaf(v[j], 1.4426950408889634f, -l2)), cg, -smg);
                if (rel >= 0 && rel < 32) {
                  const float hit = (1.f - g.smoothing) * gs;
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (j == rel) v[j] -= hit;
                }
              } else {
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
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                      if (col0 + j < g.N) v[j] += cp[j];
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
              }
            }
            // the buffer written two stores ago must have been read out by its TMA store
            if (push_base == nullptr && lane == 0) tma_store_wait_read<1>();
            __syncwarp();
            uint8_t* dstrow = stg + buf * 4096 + lane * 128;
            if (g.out_fp32) {
#pragma unroll
              for (int cc = 0; cc < 8; ++cc) {
                uint4 u = make_uint4(r[4 * cc], r[4 * cc + 1], r[4 * cc + 2], r[4 * cc + 3]);
                *reinterpret_cast<uint4*>(dstrow + ((cc ^ (lane & 7)) << 4)) = u;
              }
            } else {
#pragma unroll
              for (int cc = 0; cc < 8; ++cc) {
                uint4 u;
                u.x = pack_bf16x2(__uint_as_float(r[8 * cc + 0]), __uint_as_float(r[8 * cc + 1]));
                u.y = pack_bf16x2(__uint_as_float(r[8 * cc + 2]), __uint_as_float(r[8 * cc + 3]));
                u.z = pack_bf16x2(__uint_as_float(r[8 * cc + 4]), __uint_as_float(r[8 * cc + 5]));
                u.w = pack_bf16x2(__uint_as_float(r[8 * cc + 6]), __uint_as_float(r[8 * cc + 7]));
                *reinterpret_cast<uint4*>(dstrow + ((cc ^ (lane & 7)) << 4)) = u;
              }
            }
            if (push_base != nullptr) {
              // peer destination: plain 16-byte stores, 8 lanes per 128-byte row segment (full lines on the wire)
              __syncwarp();
              const int chunk = lane & 7;
              const int ccol = colbase + chunk * 8;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = (lane >> 3) + 4 * i;
                const int grow = row0w + rr;
                if (grow < g.M && ccol < g.N) {
                  const uint4 u = *reinterpret_cast<const uint4*>(stg + buf * 4096 + rr * 128 + ((chunk ^ (rr & 7)) << 4));
                  *reinterpret_cast<uint4*>(push_base + static_cast<long long>(grow) * g.ldc + ccol) = u;
                }
              }
              __syncwarp();
            } else {
            fence_async_smem();
            __syncwarp();
            CB_DEBUG_CHECK_ST(g.status, colbase >= 0 && row0w >= 0 && (colbase * (g.out_fp32 ? 4 : 2)) % 16 == 0,
                              CB_DBG_TMA_COORD, colbase);
            if (lane == 0 && row0w < g.M) {          // a box that starts past the last row has nothing to write
              if (g.items_per_ksplit > 0) tma_reduce_add_2d(&tmC, stg + buf * 4096, colbase, row0w);   // split K: sum the ranges
              else tma_store_2d(&tmC, stg + buf * 4096, colbase, row0w);
              tma_store_commit();
            }
            }
            buf ^= 1;
          }
        } else {
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col0 = nt * BLOCK_N + c * 32;
          if (col0 >= g.N) continue;  // uniform across the warp
          const bool full_chunk = (col0 + 32 <= g.N);

          if (EPI == EPI_LSE) {
            if (row_ok) {
              float cmax = -INFINITY;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float v = __uint_as_float(r[j]);
                if (full_chunk || col0 + j < g.N) cmax = fmaxf(cmax, v);
              }
              const float nm = fmaxf(run_m, cmax);
              const float nm2 = nm * 1.4426950408889634f;
              float acc_s = 0.f, acc_l = 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float v = __uint_as_float(r[j]);
                if (full_chunk || col0 + j < g.N) {
                  acc_s += exp2f(fmaf(v, 1.4426950408889634f, -nm2));
                  acc_l += v;
                }
              }
              run_s = run_s * exp2f((run_m - nm) * 1.4426950408889634f) + acc_s;
              run_m = nm;
              run_sum += acc_l;
              const int rel = lab - col0;
              if (rel >= 0 && rel < 32) {
                float t = 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j == rel) t = __uint_as_float(r[j]);
                g.tgt[row] = t;
              }
            }
          } else {
            if (row_ok) {
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
              if (EPI == EPI_DLOGITS) {
                const float sm = g.smoothing / static_cast<float>(g.V_total);
                const float l2 = lse_r * 1.4426950408889634f;
                const int rel = lab - col0;
                // (softmax * coef - sm) * gs as  fma, ex2, fma  per element; the label's -(1 - smoothing) * gs is
                // added afterwards by the few lanes whose label falls into these 32 columns (the epilogue warps
                // run one per scheduler, so every instruction in this loop is paid at its full latency)
                const float cg = coef * gs, smg = sm * gs;
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = fmaf(ex2_approx(fmaf(v[j], 1.4426950408889634f, -l2)), cg, -smg);
                if (rel >= 0 && rel < 32) {
                  const float hit = (1.f - g.smoothing) * gs;
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (j == rel) v[j] -= hit;
                }
              } else {
                if (g.bias != nullptr) {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (full_chunk || col0 + j < g.N) v[j] += __bfloat162float(g.bias[col0 + j]);
                }
                if (g.addend != nullptr) {
                  const bf16* ap = g.addend + static_cast<long long>(row) * g.ld_add + col0;
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (full_chunk || col0 + j < g.N) v[j] += __bfloat162float(ap[j]);
                }
              }
              if (g.out_fp32 && g.items_per_ksplit > 0) {
                float* cp = reinterpret_cast<float*>(g.C) + static_cast<long long>(row) * g.ldc + col0;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (full_chunk || col0 + j < g.N) atomicAdd(cp + j, v[j]);   // partial sums of the K ranges
              } else if (g.out_fp32) {
                float* cp = reinterpret_cast<float*>(g.C) + static_cast<long long>(row) * g.ldc + col0;
                const bool vec = full_chunk && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
                if (vec) {
                  float4* c4 = reinterpret_cast<float4*>(cp);
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    if (g.accumulate) {
                      const float4 old = c4[j];
                      o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                    }
                    c4[j] = o;
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (col0 + j < g.N) cp[j] = g.accumulate ? cp[j] + v[j] : v[j];
                }
              } else {
                bf16* cp = reinterpret_cast<bf16*>(g.C) + static_cast<long long>(row) * g.ldc + col0;
                const bool vec = full_chunk && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
                if (vec) {
                  uint4* c4 = reinterpret_cast<uint4*>(cp);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (g.accumulate) {
                      const uint4 old = c4[j];
                      const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y);
                      const float2 o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
                      v[8 * j + 0] += o0.x; v[8 * j + 1] += o0.y; v[8 * j + 2] += o1.x; v[8 * j + 3] += o1.y;
                      v[8 * j + 4] += o2.x; v[8 * j + 5] += o2.y; v[8 * j + 6] += o3.x; v[8 * j + 7] += o3.y;
                    }
                    uint4 o;
                    o.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
                    o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                    o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                    o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                    c4[j] = o;
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (col0 + j < g.N) {
                      const float o = g.accumulate ? __bfloat162float(cp[j]) + v[j] : v[j];
                      cp[j] = __float2bfloat16(o);
                    }
                }
              }
            }
          }
        }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty + acc);
      }
      if (EPI == EPI_LSE && ok && row_ok) {
        const long long o = static_cast<long long>(split) * g.M + row;
        g.part_m[o] = run_m;
        g.part_s[o] = run_s;
        if (g.part_sum != nullptr) g.part_sum[o] = run_sum;
      }
    }
    if (EPI != EPI_LSE && g.tma_store && lane == 0) tma_store_wait_all();
  }

  // ------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {
    // a wait was abandoned: give copies already in flight time to land before the smem is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ combine kernels for cut-cross-entropy
// lse[row] from the per-split partials; per-row loss with smoothing and z-loss.
__global__ void cce_combine_rows_kernel(const float* __restrict__ part_m, const float* __restrict__ part_s,
                                        const float* __restrict__ part_sum, const float* __restrict__ tgt,
                                        const long long* __restrict__ labels, int M, int n_splits, int V_total,
                                        float smoothing, float z_weight, long long ignore_index,
                                        float* __restrict__ lse_out, float* __restrict__ loss_rows) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_m[static_cast<long long>(s) * M + row]);
  float sum = 0.f, sl = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const long long o = static_cast<long long>(s) * M + row;
    const float pm = part_m[o];
    if (pm > -INFINITY) sum += part_s[o] * __expf(pm - m);
    if (part_sum != nullptr) sl += part_sum[o];
  }
  const float lse = m + __logf(sum);
  lse_out[row] = lse;
  const bool valid = labels[row] != ignore_index;
  float loss = lse - tgt[row];
  if (smoothing != 0.f) loss = (1.f - smoothing) * loss + smoothing * (lse - sl / static_cast<float>(V_total));
  loss += z_weight * lse * lse;
  loss_rows[row] = valid ? loss : 0.f;
}

// Single block: deterministic sum of per-row losses and the valid count; writes
// out[0] = mean (or sum), out[1] = n_valid, and gscale[row] = valid / n_valid (or valid).
__global__ void cce_finalize_kernel(const float* __restrict__ loss_rows, const long long* __restrict__ labels, int M,
                                    long long ignore_index, int mean, float* __restrict__ out,
                                    float* __restrict__ gscale) {
  __shared__ float s_sum[32];
  __shared__ float s_cnt[32];
  __shared__ float s_n;
  float sum = 0.f, cnt = 0.f;
  for (int i = threadIdx.x; i < M; i += blockDim.x) {
    sum += loss_rows[i];
    cnt += (labels[i] != ignore_index) ? 1.f : 0.f;
  }
  sum = warp_sum(sum);
  cnt = warp_sum(cnt);
  if ((threadIdx.x & 31) == 0) {
    s_sum[threadIdx.x >> 5] = sum;
    s_cnt[threadIdx.x >> 5] = cnt;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    float a = threadIdx.x < nw ? s_sum[threadIdx.x] : 0.f;
    float b = threadIdx.x < nw ? s_cnt[threadIdx.x] : 0.f;
    a = warp_sum(a);
    b = warp_sum(b);
    if (threadIdx.x == 0) {
      const float n = fmaxf(b, 1.f);
      out[0] = mean ? a / n : a;
      out[1] = b;
      s_n = mean ? n : 1.f;
    }
  }
  __syncthreads();
  const float inv = 1.f / s_n;
  for (int i = threadIdx.x; i < M; i += blockDim.x) gscale[i] = (labels[i] != ignore_index) ? inv : 0.f;
}

}  // namespace cb

// =========================================================================================== host side
extern "C" int cb_gemm2sm_supported(const void* C, long long ldc, int out_fp32);
extern "C" int cb_gemm2sm_cost_milli(int M, int N, int K, int pairs_avail);
extern "C" int cb_gemm2sm_bf16(const void* A, const void* B, void* C, const void* bias, const void* addend, int M, int N,
                               int K, long long lda, long long ldb, long long ldc, long long ld_add, int a_mn, int b_mn,
                               int out_fp32, int accumulate, int* status, void* stream);

namespace {

using cbhost::make_tmap;
using cbhost::num_sms;

template <int BLOCK_N, int A_MN, int B_MN, int STAGES, int EPI>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const cb::GemmArgs& g,
           cudaStream_t stream) {
  auto kern = cb::gemm_tcgen05_kernel<BLOCK_N, A_MN, B_MN, STAGES, EPI>;
  constexpr int smem = cb::SmemLayout<BLOCK_N, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    CB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  const int grid = g.num_items < num_sms() ? g.num_items : num_sms();
  kern<<<grid, cb::GEMM_THREADS, smem, stream>>>(ta, tb, tc, g);
  return static_cast<int>(cudaGetLastError());
}

template <int EPI>
int dispatch(int block_n, int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
             const cb::GemmArgs& g, cudaStream_t s) {
  if (block_n == 256) {
    if (!a_mn && !b_mn) return launch<256, 0, 0, 4, EPI>(ta, tb, tc, g, s);
    if (EPI == cb::EPI_STORE) {
      if (!a_mn && b_mn) return launch<256, 0, 1, 4, cb::EPI_STORE>(ta, tb, tc, g, s);
      if (a_mn && b_mn) return launch<256, 1, 1, 4, cb::EPI_STORE>(ta, tb, tc, g, s);
      if (a_mn && !b_mn) return launch<256, 1, 0, 4, cb::EPI_STORE>(ta, tb, tc, g, s);
    }
  } else {
    if (!a_mn && !b_mn) return launch<128, 0, 0, 6, EPI>(ta, tb, tc, g, s);
    if (EPI == cb::EPI_STORE) {
      if (!a_mn && b_mn) return launch<128, 0, 1, 6, cb::EPI_STORE>(ta, tb, tc, g, s);
      if (a_mn && b_mn) return launch<128, 1, 1, 6, cb::EPI_STORE>(ta, tb, tc, g, s);
      if (a_mn && !b_mn) return launch<128, 1, 0, 6, cb::EPI_STORE>(ta, tb, tc, g, s);
    }
  }
  return -20;
}

int pick_block_n(int M, int N, int forced) {
  if (forced == 128 || forced == 256) return forced;
  const int mb = (M + 127) / 128;
  const int sms = num_sms();
  long long best_cost = -1;
  int best = 256;
  for (int bn : {256, 128}) {
    const long long tiles = static_cast<long long>(mb) * ((N + bn - 1) / bn);
    const long long waves = (tiles + sms - 1) / sms;
    const long long cost = waves * (bn + 24);  // +24: per-tile fixed overhead in the same unit
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

// Time of each kernel in units of one round of 256 x 256 CTA-pair tiles.  The pair kernel balances a partial last
// round by cutting tiles along K (its own estimate, cb_gemm2sm_cost_milli); the single-CTA kernels run whole
// tiles only (measured on the 0.5B shapes: a 128x256 round takes ~1.08 pair rounds, a 128x128 round ~0.9 because
// those tiles are bound by operand bandwidth, not by the tensor pipe).  Short GEMMs stay on the single-CTA
// kernel, whose fixed costs are lower.
bool prefer_cta_pairs(int M, int N, int K) {
  if (K < 1024 && N < 1024) return false;
  const int sms = num_sms();
  const long long t256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256);
  const long long t128 = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128);
  const double c2 = cb_gemm2sm_cost_milli(M, N, K, sms / 2) / 1000.0;
  const double c256 = 1.08 * static_cast<double>((t256 + sms - 1) / sms);
  const double c128 = 0.90 * static_cast<double>((t128 + sms - 1) / sms);
  return c2 <= (c256 < c128 ? c256 : c128);
}

// Tensor map of the output for the staged epilogue; returns 0 and sets *ok when C qualifies
// (16-byte aligned base and row pitch), otherwise leaves the direct-store epilogue in charge.
int build_out_map(CUtensorMap* tc, int* ok, const void* C, int M, int N, long long ldc, int out_fp32) {
  const int eb = out_fp32 ? 4 : 2;
  *ok = 0;
  memset(tc, 0, sizeof(*tc));
  if ((reinterpret_cast<uintptr_t>(C) & 15) != 0 || (ldc * eb) % 16 != 0) return 0;
  const int e = make_tmap(tc, C, N, M, ldc, out_fp32 ? 32 : 64, 32, eb);
  if (e) return e;
  *ok = 1;
  return 0;
}

int build_maps(CUtensorMap* ta, CUtensorMap* tb, const void* A, const void* B, int M, int N, int K, long long lda,
               long long ldb, int a_mn, int b_mn, int block_n) {
  int e;
  if (!a_mn) e = make_tmap(ta, A, K, M, lda, 64, cb::BLOCK_M);   // rows = M, K contiguous
  else e = make_tmap(ta, A, M, K, lda, 64, 64);                   // rows = K, M contiguous
  if (e) return e;
  if (!b_mn) e = make_tmap(tb, B, K, N, ldb, 64, block_n);
  else e = make_tmap(tb, B, N, K, ldb, 64, 64);
  return e;
}

}  // namespace

extern "C" {

// C[M,N] = A * B^T (+bias) (+addend) (+C).  a_mn / b_mn: 0 when the operand is stored [M|N, K]
// (K contiguous), 1 when stored [K, M|N].  lda/ldb/ldc/ld_add are row pitches in elements.
// Returns 0 on a successful launch; negative for rejected arguments; positive CUDA error otherwise.
int cb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* addend, int M, int N, int K,
                 long long lda, long long ldb, long long ldc, long long ld_add, int a_mn, int b_mn, int out_fp32,
                 int accumulate, int force_block_n, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  // force_block_n: 0 = choose (CTA-pair kernel or 128 / 256 wide single-CTA tiles), 128 / 256 = single-CTA tile
  // of that width, 2 = CTA-pair kernel
  if ((force_block_n == 2 || (force_block_n == 0 && prefer_cta_pairs(M, N, K))) && cb_gemm2sm_supported(C, ldc, out_fp32))
    return cb_gemm2sm_bf16(A, B, C, bias, addend, M, N, K, lda, ldb, ldc, ld_add, a_mn, b_mn, out_fp32, accumulate,
                           status, stream);
  if (force_block_n == 2) force_block_n = 0;
  const int bn = pick_block_n(M, N, force_block_n);
  CUtensorMap ta, tb;
  int e = build_maps(&ta, &tb, A, B, M, N, K, lda, ldb, a_mn, b_mn, bn);
  if (e) return e;
  cb::GemmArgs g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_blocks = (M + 127) / 128;
  g.num_n_tiles = (N + bn - 1) / bn;
  g.tiles_per_item = 1;
  g.num_items = g.num_m_blocks * g.num_n_tiles;
  g.C = C; g.ldc = ldc; g.out_fp32 = out_fp32; g.accumulate = accumulate;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.addend = static_cast<const cb::bf16*>(addend);
  g.ld_add = ld_add;
  g.status = status;
  CUtensorMap tc;
  e = build_out_map(&tc, &g.tma_store, C, M, N, ldc, out_fp32);
  if (e) return e;
  return dispatch<cb::EPI_STORE>(bn, a_mn, b_mn, ta, tb, tc, g, static_cast<cudaStream_t>(stream));
}

// Split-K GEMM for skinny outputs: C[M,N] (fp32, zeroed here) = A * B^T with the K range cut into pieces so
// that about one CTA per SM is busy even when the output has only a few tiles (weight gradients of low-rank
// adapters: M or N of 16..64 with K = tokens).  Partial tiles are summed with red.global.add.
int cb_gemm_bf16_splitk(const void* A, const void* B, float* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  const int bn = 128;
  CUtensorMap ta, tb, tc;
  int e = build_maps(&ta, &tb, A, B, M, N, K, lda, ldb, a_mn, b_mn, bn);
  if (e) return e;
  memset(&tc, 0, sizeof(tc));
  cb::GemmArgs g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_blocks = (M + 127) / 128;
  g.num_n_tiles = (N + bn - 1) / bn;
  g.tiles_per_item = 1;
  const int tiles = g.num_m_blocks * g.num_n_tiles;
  const int num_kb = (K + 63) / 64;
  int splits = num_sms() / tiles;
  if (splits < 1) splits = 1;
  if (splits > num_kb) splits = num_kb;
  g.kb_per_split = (num_kb + splits - 1) / splits;
  splits = (num_kb + g.kb_per_split - 1) / g.kb_per_split;
  g.items_per_ksplit = tiles;
  g.num_items = tiles * splits;
  g.C = C; g.ldc = ldc; g.out_fp32 = 1;
  g.tma_store = 0;
  if ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * 4) % 16 == 0) {
    // partial tiles go through the staging buffers and are added into C by TMA reduce (128-byte rows of 32 floats);
    // otherwise each thread adds its elements one by one
    e = cbhost::make_tmap(&tc, C, N, M, ldc, 32, 32, 4);
    if (e) return e;
    g.tma_store = 1;
  }
  g.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CB_CHECK_CUDA(cudaMemset2DAsync(C, sizeof(float) * ldc, 0, sizeof(float) * N, M, s));
  return dispatch<cb::EPI_STORE>(bn, a_mn, b_mn, ta, tb, tc, g, s);
}

// Tensor-parallel variants of cb_gemm_bf16 (bf16 output, no addend / accumulate).
//  * panel_rows > 0 (all-gather -> GEMM): A's rows arrive in W panels of panel_rows rows pushed by the peers;
//    panel_flags[src] (local, u64) reaches *panel_epoch when panel src is complete.  The kernel starts with
//    this rank's own panel and waits (bounded by wait_ns) per panel while the others are still in flight.
//  * push_rows > 0 (GEMM -> reduce-scatter): output rows [o * push_rows, (o + 1) * push_rows) are stored
//    through push_ptrs[o] (peer mappings, host array of W addresses, pre-offset so that the global row
//    number indexes them with pitch ldc); C is ignored.
// panel_rows and push_rows must be multiples of 128; with push, N and ldc must be multiples of 8.
int cb_gemm_bf16_tp(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int a_mn, int b_mn, int force_block_n,
                    const unsigned long long* panel_flags, const unsigned long long* panel_epoch, int panel_rows,
                    const unsigned long long* push_ptrs, int push_rows, int W, int my_rank,
                    unsigned long long wait_ns, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || W < 1 || W > 16 || my_rank < 0 || my_rank >= W) return -1;
  if (panel_rows < 0 || push_rows < 0 || panel_rows % 128 != 0 || push_rows % 128 != 0) return -2;
  if (panel_rows > 0 && (panel_flags == nullptr || panel_epoch == nullptr || panel_rows * W < M)) return -3;
  if (push_rows > 0 && (push_ptrs == nullptr || push_rows * W < M || N % 8 != 0 || ldc % 8 != 0)) return -4;
  const int bn = pick_block_n(M, N, force_block_n);
  CUtensorMap ta, tb;
  int e = build_maps(&ta, &tb, A, B, M, N, K, lda, ldb, a_mn, b_mn, bn);
  if (e) return e;
  cb::GemmArgs g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_blocks = (M + 127) / 128;
  g.num_n_tiles = (N + bn - 1) / bn;
  g.tiles_per_item = 1;
  g.num_items = g.num_m_blocks * g.num_n_tiles;
  g.C = C; g.ldc = ldc;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.status = status;
  g.peer_wait_ns = wait_ns;
  CUtensorMap tc;
  memset(&tc, 0, sizeof(tc));
  if (panel_rows > 0) {
    g.panel_flags = panel_flags;
    g.panel_epoch = panel_epoch;
    g.panel_blocks = panel_rows / 128;
    g.panel_self = my_rank;
    g.rot_blocks = (my_rank * g.panel_blocks) % g.num_m_blocks;
  }
  if (push_rows > 0) {
    g.push_blocks = push_rows / 128;
    for (int i = 0; i < W; ++i) g.push_c[i] = push_ptrs[i];
    g.rot_blocks = (my_rank * g.push_blocks) % g.num_m_blocks;
    g.tma_store = 1;           // staged epilogue; the tile leaves shared memory by plain stores to the peer
    g.C = nullptr;
  } else {
    e = build_out_map(&tc, &g.tma_store, C, M, N, ldc, 0);
    if (e) return e;
  }
  return dispatch<cb::EPI_STORE>(bn, a_mn, b_mn, ta, tb, tc, g, static_cast<cudaStream_t>(stream));
}

// Number of vocab splits the forward pass of the fused linear-cross-entropy uses for a
// [M, V] problem (the partial buffers are [n_splits, M]).
int cb_cce_num_splits(int M, int V) {
  const int tiles = (V + 255) / 256;
  const int per = tiles < 16 ? tiles : 16;
  return (tiles + per - 1) / per;
}

// Forward: per-row log-sum-exp partials of hidden[M,K] * weight[V,K]^T, target logit.
int cb_cce_forward(const void* hidden, const void* weight, const long long* labels, int M, int V, int K,
                   long long ldh, long long ldw, int col_offset, float* part_m, float* part_s, float* part_sum,
                   float* tgt, int* status, void* stream) {
  const int bn = 256;
  CUtensorMap ta, tb;
  int e = build_maps(&ta, &tb, hidden, weight, M, V, K, ldh, ldw, 0, 0, bn);
  if (e) return e;
  cb::GemmArgs g = {};
  g.M = M; g.N = V; g.K = K;
  g.num_m_blocks = (M + 127) / 128;
  g.num_n_tiles = (V + bn - 1) / bn;
  g.tiles_per_item = g.num_n_tiles < 16 ? g.num_n_tiles : 16;
  const int n_splits = (g.num_n_tiles + g.tiles_per_item - 1) / g.tiles_per_item;
  g.num_items = g.num_m_blocks * n_splits;
  g.labels = labels;
  g.part_m = part_m; g.part_s = part_s; g.part_sum = part_sum; g.tgt = tgt;
  g.col_offset = col_offset;
  g.status = status;
  CUtensorMap tc;
  memset(&tc, 0, sizeof(tc));
  return dispatch<cb::EPI_LSE>(bn, 0, 0, ta, tb, tc, g, static_cast<cudaStream_t>(stream));
}

int cb_cce_combine(const float* part_m, const float* part_s, const float* part_sum, const float* tgt,
                   const long long* labels, int M, int n_splits, int V_total, float smoothing, float z_weight,
                   long long ignore_index, int mean, float* lse, float* loss_rows, float* out, float* gscale,
                   void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cb::cce_combine_rows_kernel<<<(M + 255) / 256, 256, 0, s>>>(part_m, part_s, part_sum, tgt, labels, M, n_splits,
                                                              V_total, smoothing, z_weight, ignore_index, lse,
                                                              loss_rows);
  cb::cce_finalize_kernel<<<1, 1024, 0, s>>>(loss_rows, labels, M, ignore_index, mean, out, gscale);
  return static_cast<int>(cudaGetLastError());
}

// Backward, step 1: G[M, Vc] = d(loss)/d(logits) for the vocab columns [col_offset, col_offset + Vc)
// of `weight_chunk` (= weight + col_offset * ldw), written as bf16 with row pitch ldg.
int cb_cce_dlogits(const void* hidden, const void* weight_chunk, const long long* labels, const float* lse,
                   const float* gscale, const float* gout, void* G, int M, int Vc, int K, long long ldh,
                   long long ldw, long long ldg, int col_offset, int V_total, float smoothing, float z_weight,
                   int* status, void* stream) {
  const int bn = pick_block_n(M, Vc, 0);
  CUtensorMap ta, tb;
  int e = build_maps(&ta, &tb, hidden, weight_chunk, M, Vc, K, ldh, ldw, 0, 0, bn);
  if (e) return e;
  cb::GemmArgs g = {};
  g.M = M; g.N = Vc; g.K = K;
  g.num_m_blocks = (M + 127) / 128;
  g.num_n_tiles = (Vc + bn - 1) / bn;
  g.tiles_per_item = 1;
  g.num_items = g.num_m_blocks * g.num_n_tiles;
  g.C = G; g.ldc = ldg; g.out_fp32 = 0; g.accumulate = 0;
  g.labels = labels; g.lse = lse; g.gscale = gscale; g.gout = gout;
  g.z_weight = z_weight; g.smoothing = smoothing; g.V_total = V_total; g.col_offset = col_offset;
  g.status = status;
  CUtensorMap tc;
  e = build_out_map(&tc, &g.tma_store, G, M, Vc, ldg, 0);
  if (e) return e;
  return dispatch<cb::EPI_DLOGITS>(bn, 0, 0, ta, tb, tc, g, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
