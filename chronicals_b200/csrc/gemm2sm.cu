// Two-CTA tcgen05 GEMM: C[M,N] = A[M,K] * B[N,K]^T (bf16 in / out, fp32 accumulation) with one
// 256 x 256 output tile per CTA pair (`tcgen05.mma.cta_group::2`).
//
// Why: with one CTA per tile (gemm.cu, 128 x 256) every k-block of 64 needs 48 KB of operands per 512 MMA
// cycles and SM; the shared-memory ring then holds about one memory latency of data and every L2 miss reaches
// the MMA issuer.  A CTA pair shares the B tile: each CTA loads its own 128 rows of A and only HALF of the
// 256 rows of B (32 KB per k-block and SM), the tensor cores of both SMs read the two halves from both
// shared memories, and the ring is six stages deep instead of four.
//
// Structure (192 threads per CTA, cluster of 2 along x):
//   warp 0      TMA producer of this CTA's A rows and B half (ordinary, non-multicast TMA loads into the CTA's
//               own shared memory, signalling the CTA's own `full` barrier)
//   warp 1      leader CTA (rank 0): issues the MMAs for the pair once its own stage AND the peer's stage are
//               full; `tcgen05.commit ... multicast::cluster` releases the stage / publishes the accumulator in
//               both CTAs.  Peer CTA (rank 1): relays "my stage is full" to the leader with a remote mbarrier
//               arrive.
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
constexpr int BN = 256;          // columns of the pair's tile
constexpr int BNH = 128;         // rows of B loaded by each CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STG_OFFSET = STAGES * (A_BYTES + B_BYTES);
constexpr int BAR_OFFSET = STG_OFFSET + 4 * 8192;
constexpr int SMEM_TOTAL = BAR_OFFSET + 512 + 1024;

struct Args {
  int M, N, K;
  int num_m_pairs, num_n_tiles, num_tiles;
  void* C;                 // output (needed for accumulate; the stores go through the tensor map)
  long long ldc;
  int out_fp32;
  int accumulate;
  const bf16* bias;        // [N] or null
  const bf16* addend;      // [M, N] with row pitch ld_add, or null (residual)
  long long ld_add;
  const float* row_scale;  // fp8 operands: C = (A_q B_q^T) * row_scale[m] * col_scale[n]; null for bf16 operands
  const float* col_scale;
  int* status;
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

// A_MN / B_MN: 0 = operand stored [rows, K] (K contiguous), 1 = stored [K, rows] (rows contiguous), exactly as in
// gemm.cu, so forward (0,0), dgrad (0,1) and wgrad (1,1) need no transposed copies.
// KIND: 0 = bf16 operands (kind::f16, 64 elements per k-block), 1 = e4m3 operands (kind::f8f6f4, 128 elements per
// k-block, K-major only).  Either way a k-block row is 128 bytes and one MMA consumes 32 bytes of it, so the
// shared-memory layout, the descriptors and the pipeline are identical.
template <int NACC, int A_MN, int B_MN, int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const Args g) {
  constexpr uint32_t TMEM_COLS = NACC * BN;                              // NACC accumulators of 256 columns
  constexpr uint32_t IDESC = KIND ? umma_idesc_fp8(2 * BM, BN, 0, 0)
                                  : umma_idesc_bf16(2 * BM, BN, A_MN, B_MN);      // M = 256 across the pair
  constexpr int BKE = KIND ? 2 * BK : BK;                                // elements per k-block

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + BAR_OFFSET);       // my TMA stage landed
  uint64_t* peer_full = full + STAGES;                                   // (leader) the peer's stage landed
  uint64_t* empty = peer_full + STAGES;                                  // stage consumed (multicast commit)
  uint64_t* tfull = empty + STAGES;                                      // accumulator complete (multicast commit)
  uint64_t* tempty = tfull + 2;                                          // (leader) accumulator drained by both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(peer_full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < NACC; ++a) {
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
  const int num_kb = (g.K + BKE - 1) / BKE;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (each CTA: its A rows, its B half)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < g.num_tiles && ok; t += num_pairs) {
        const int mp = t % g.num_m_pairs;
        const int nt = t / g.num_m_pairs;
        const int a_row = mp * 2 * BM + static_cast<int>(rank) * BM;
        const int b_row = nt * BN + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(full + stage, A_BYTES + B_BYTES);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (A_MN == 0) {
            tma_load_2d(a_dst, &tmA, full + stage, kb * BKE, a_row);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, full + stage, a_row + j * 64, kb * BK);
          }
          if (B_MN == 0) {
            tma_load_2d(b_dst, &tmB, full + stage, kb * BKE, b_row);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, full + stage, b_row + j * 64, kb * BK);
          }
          if (++stage == STAGES) {
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
        // --------------------------------------------------------- MMA issuer for the pair
        uint32_t tile_cnt = 0;
        for (int t = pair; t < g.num_tiles && ok; t += num_pairs, ++tile_cnt) {
          const uint32_t acc = tile_cnt % NACC;
          const uint32_t acc_phase = (tile_cnt / NACC) & 1u;
          if (!mbar_wait(tempty + acc, acc_phase ^ 1, abort_flag, g.status, CB_ERR_WAIT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_FULL) ||
                !mbar_wait(peer_full + stage, phase, abort_flag, g.status, CB_ERR_WAIT_PEER)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_base = smem_u32(sA + stage * A_BYTES);
            const uint32_t b_base = smem_u32(sB + stage * B_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t adesc = A_MN ? umma_smem_desc(a_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc(a_base + k * 32, 16, 1024);
              const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc(b_base + k * 32, 16, 1024);
              if (KIND) umma_f8_ss_2cta(d_tmem, adesc, bdesc, IDESC, (kb | k) != 0 ? 1u : 0u);
              else umma_f16_ss_2cta(d_tmem, adesc, bdesc, IDESC, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit_2cta(empty + stage);      // frees this stage in both CTAs once the MMAs retire
            if (++stage == STAGES) {
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
            if (++stage == STAGES) {
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
    uint8_t* stg = smem + STG_OFFSET + (warp - 2) * 8192;
    uint32_t tile_cnt = 0;
    bool ok = true;
    for (int t = pair; t < g.num_tiles && ok; t += num_pairs, ++tile_cnt) {
      const int mp = t % g.num_m_pairs;
      const int nt = t / g.num_m_pairs;
      const uint32_t acc = tile_cnt % NACC;
      const uint32_t acc_phase = (tile_cnt / NACC) & 1u;
      bool w = mbar_wait(tfull + acc, acc_phase, abort_flag, g.status, CB_ERR_WAIT_TMEM_FULL);
      w = __all_sync(0xffffffffu, w);
      if (!w) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int row0w = mp * 2 * BM + static_cast<int>(rank) * BM + q * 32;
      const int row = row0w + lane;
      const bool row_ok = row < g.M;
      const int cols_per_store = g.out_fp32 ? 32 : 64;
      int buf = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += cols_per_store) {
        const int colbase = nt * BN + c0;
        if (colbase >= g.N) break;                          // uniform across the warp
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
        }
        if (lane == 0) tma_store_wait_read<1>();            // the buffer written two stores ago has been read out
        __syncwarp();
        uint8_t* dstrow = stg + buf * 4096 + lane * 128;
        if (g.out_fp32) {
#pragma unroll
          for (int cc = 0; cc < 8; ++cc) {
            const uint4 u = make_uint4(r[4 * cc], r[4 * cc + 1], r[4 * cc + 2], r[4 * cc + 3]);
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
        fence_async_smem();
        __syncwarp();
        if (lane == 0 && row0w < g.M) {                      // a box that starts past the last row has nothing to write
          tma_store_2d(&tmC, stg + buf * 4096, colbase, row0w);
          tma_store_commit();
        }
        buf ^= 1;
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

}  // namespace cb2

namespace {

template <int A_MN, int B_MN, int KIND = 0>
int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const cb2::Args& g, cudaStream_t s) {
  auto kern = cb2::gemm2sm_kernel<2, A_MN, B_MN, KIND>;
  static bool configured = false;
  if (!configured) {
    CB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cb2::SMEM_TOTAL));
    configured = true;
  }
  int pairs = cbhost::num_sms() / 2;
  if (pairs > g.num_tiles) pairs = g.num_tiles;
  kern<<<2 * pairs, cb2::THREADS, cb2::SMEM_TOTAL, s>>>(ta, tb, tc, g);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

// Whether cb_gemm2sm_bf16 can take this problem (TMA-store epilogue needs an aligned C and pitch).
int cb_gemm2sm_supported(const void* C, long long ldc, int out_fp32) {
  const int eb = out_fp32 ? 4 : 2;
  return ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * eb) % 16 == 0) ? 1 : 0;
}

// C[M,N] = op(A) * op(B)^T (+bias) (+addend) (+C) on CTA pairs.  Same conventions as cb_gemm_bf16 (gemm.cu):
// a_mn / b_mn = 0 for operands stored [rows, K], 1 for [K, rows]; pitches in elements.
int cb_gemm2sm_bf16(const void* A, const void* B, void* C, const void* bias, const void* addend, int M, int N, int K,
                    long long lda, long long ldb, long long ldc, long long ld_add, int a_mn, int b_mn, int out_fp32,
                    int accumulate, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (!cb_gemm2sm_supported(C, ldc, out_fp32)) return -2;
  CUtensorMap ta, tb, tc;
  int e;
  if (!a_mn) e = cbhost::make_tmap(&ta, A, K, M, lda, 64, cb2::BM);
  else e = cbhost::make_tmap(&ta, A, M, K, lda, 64, 64);
  if (e) return e;
  if (!b_mn) e = cbhost::make_tmap(&tb, B, K, N, ldb, 64, cb2::BNH);
  else e = cbhost::make_tmap(&tb, B, N, K, ldb, 64, 64);
  if (e) return e;
  e = cbhost::make_tmap(&tc, C, N, M, ldc, out_fp32 ? 32 : 64, 32, out_fp32 ? 4 : 2);
  if (e) return e;
  cb2::Args g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_pairs = (M + 2 * cb2::BM - 1) / (2 * cb2::BM);
  g.num_n_tiles = (N + cb2::BN - 1) / cb2::BN;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.C = C; g.ldc = ldc; g.out_fp32 = out_fp32; g.accumulate = accumulate;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.addend = static_cast<const cb::bf16*>(addend);
  g.ld_add = ld_add;
  g.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch2<0, 0>(ta, tb, tc, g, s);
  if (!a_mn && b_mn) return launch2<0, 1>(ta, tb, tc, g, s);
  if (a_mn && b_mn) return launch2<1, 1>(ta, tb, tc, g, s);
  return launch2<1, 0>(ta, tb, tc, g, s);
}


// FP8 (e4m3) GEMM on the tensor cores: C[M,N] (bf16) = (Aq[M,K] * Bq[N,K]^T) * row_scale[m] * col_scale[n] (+bias).
// Aq / Bq hold e4m3 bytes with K contiguous; pitches in bytes, multiples of 16; K a multiple of 16.
int cb_gemm2sm_fp8(const void* Aq, const void* Bq, void* C, const float* row_scale, const float* col_scale,
                   const void* bias, int M, int N, int K, long long lda, long long ldb, long long ldc, int* status,
                   void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 16 != 0 || row_scale == nullptr || col_scale == nullptr) return -1;
  if (!cb_gemm2sm_supported(C, ldc, 0)) return -2;
  CUtensorMap ta, tb, tc;
  int e = cbhost::make_tmap(&ta, Aq, K, M, lda, 128, cb2::BM, 1);
  if (e) return e;
  e = cbhost::make_tmap(&tb, Bq, K, N, ldb, 128, cb2::BNH, 1);
  if (e) return e;
  e = cbhost::make_tmap(&tc, C, N, M, ldc, 64, 32, 2);
  if (e) return e;
  cb2::Args g = {};
  g.M = M; g.N = N; g.K = K;
  g.num_m_pairs = (M + 2 * cb2::BM - 1) / (2 * cb2::BM);
  g.num_n_tiles = (N + cb2::BN - 1) / cb2::BN;
  g.num_tiles = g.num_m_pairs * g.num_n_tiles;
  g.C = C; g.ldc = ldc;
  g.bias = static_cast<const cb::bf16*>(bias);
  g.row_scale = row_scale;
  g.col_scale = col_scale;
  g.status = status;
  return launch2<0, 0, 1>(ta, tb, tc, g, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
