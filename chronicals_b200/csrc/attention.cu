// Varlen causal GQA flash attention, forward and backward, on tcgen05 tensor
// cores with the score tiles in TMEM.
//
// Layout: q [T, hq, D], k/v [T, hk, D] packed tokens (any row pitch, so they may
// be slices of one fused QKV buffer); documents are the intervals of
// cu_seqlens.  One CTA owns one 128-row block of one document and one query
// head.  Every thread owns one row of the 128 x 128 score tile: it reads its row
// from TMEM with tcgen05.ld, so the online softmax needs no cross-thread
// shuffles, and writes P (bf16) into shared memory in the 128-byte-swizzled
// layout the next MMA consumes.
//
//   forward : S = Q K^T -> P = softmax -> O += P V        (2 MMAs per kv block)
//   backward: S, dP = dO V^T -> P, dS -> dV += P^T dO, dK += dS^T Q, dQ = dS K
//
// The same swizzled image of a [128 x 64] bf16 tile serves as a K-major operand
// (rows = M/N) and as an MN-major operand (rows = K), so P^T and dS^T need no
// transposed copy.  All tensor maps cover this GPU's own memory only.
//
// Replaces the reference's calls into flash-attn / SDPA (chronicals/kernels/
// flash_attention_optimizer.py:845-994) and its forward-only Triton kernels
// (:2460-3209); the reference has no attention backward of its own.
#include <cstdlib>
#include "common.cuh"

namespace cb {

constexpr int ATT_THREADS = 128;
constexpr int BWD2_THREADS = 256;   // backward variant with two threads per score row
constexpr float LOG2E = 1.4426950408889634f;

struct AttnArgs {
  int T, hq, hk, n_docs;
  const int* cu;        // [n_docs + 1]
  float scale;
  bf16* O;              // [T, hq, D], row pitch ldo
  long long ldo;
  float* lse;           // [hq, T]
  // backward
  const float* delta;   // [hq, T]  rowsum(dO * O)
  float* dq_acc;        // [T, hq, D] fp32, zero-initialised; accumulated with red.add
  float* dk_part;       // [T, hk, D] fp32, zero-initialised; accumulated with red.add over the group's query heads
  float* dv_part;
  int* status;
};

// which (document, block) a CTA owns; blocks of one document are handed out heaviest first
__device__ __forceinline__ bool locate_block(const int* cu, int n_docs, int b, int& start, int& len, int& blk, int& nblk) {
  for (int i = 0; i < n_docs; ++i) {
    const int s = cu[i], e = cu[i + 1];
    const int nb = (e - s + 127) >> 7;
    if (b < nb) {
      start = s; len = e - s; nblk = nb; blk = b;
      return true;
    }
    b -= nb;
  }
  return false;
}

// store 32 consecutive values of thread-row r as bf16 into a [128 x 128] operand image made of two
// 64-column panels of 16 KB, 128-byte rows, 16-byte chunks XOR-swizzled by (row & 7)
__device__ __forceinline__ void store_row_chunk32(uint8_t* base, int r, int c32, const float (&v)[32]) {
  const int panel = c32 >> 1;                 // chunks 0,1 -> panel 0 ; 2,3 -> panel 1
  uint8_t* row = base + panel * 16384 + r * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int cc = (c32 & 1) * 4 + q;         // 16-byte chunk index within the 128-byte row
    uint4 u;
    u.x = pack_bf16x2(v[8 * q + 0], v[8 * q + 1]);
    u.y = pack_bf16x2(v[8 * q + 2], v[8 * q + 3]);
    u.z = pack_bf16x2(v[8 * q + 4], v[8 * q + 5]);
    u.w = pack_bf16x2(v[8 * q + 6], v[8 * q + 7]);
    *reinterpret_cast<uint4*>(row + ((cc ^ (r & 7)) << 4)) = u;
  }
}

// descriptors over a [128 rows x D] bf16 tile stored as D/64 panels of 16 KB
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int kk) {      // K = columns, k-step of 16 columns
  return umma_smem_desc(base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int kk) {     // K = rows, k-step of 16 rows
  return umma_smem_desc(base + kk * 2048, 16384, 1024);
}

// Forward softmax passes over my row of the score tile (fp32, TMEM columns [0, 128)), in two versions: the
// diagonal block masks columns beyond the row, every other block of a causal document needs no mask at all
// (7 of 8 blocks at 1024 tokens), so the common path carries no compare / select per element.
// Both passes keep the TMEM load of the next 32-column chunk in flight while they work on the current one.
template <bool DIAG>
__device__ __forceinline__ float fwd_row_max(uint32_t t_row, int r) {
  float mx = -INFINITY;
  uint32_t s[2][32];
  tmem_ld_32x32(t_row, s[0]);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (c + 1 < 4) tmem_ld_32x32(t_row + (c + 1) * 32, s[(c + 1) & 1]);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float v = __uint_as_float(s[c & 1][i]);
      if (!DIAG || c * 32 + i <= r) mx = fmaxf(mx, v);
    }
    if (c + 1 < 4) tmem_ld_wait();
  }
  return mx;
}
// P = 2^(S * sl2 - mb) written as bf16 pairs over the consumed S columns; returns the row sum
template <bool DIAG>
__device__ __forceinline__ float fwd_row_exp(uint32_t t_row, int r, float sl2, float mb) {
  float rs = 0.f;
  uint32_t s[2][32];
  tmem_ld_32x32(t_row, s[0]);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    // the chunk fetched here ([32(c+1), 32(c+2))) lies above every word written below ([16c, 16c + 16))
    if (c + 1 < 4) tmem_ld_32x32(t_row + (c + 1) * 32, s[(c + 1) & 1]);
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float e0 = ex2_approx(fmaf(__uint_as_float(s[c & 1][2 * i]), sl2, -mb));
      float e1 = ex2_approx(fmaf(__uint_as_float(s[c & 1][2 * i + 1]), sl2, -mb));
      if (DIAG) {
        e0 = (c * 32 + 2 * i <= r) ? e0 : 0.f;
        e1 = (c * 32 + 2 * i + 1 <= r) ? e1 : 0.f;
      }
      rs += e0 + e1;
      pk[i] = pack_bf16x2(e0, e1);
    }
    if (c + 1 < 4) tmem_ld_wait();
    // 32 probabilities -> 16 bf16 pairs -> TMEM words [16c, 16c + 16) of my row: always behind the
    // fp32 columns [32c, 32c + 32) already read, so S is consumed before it is overwritten
    tmem_st_32x16(t_row + c * 16, pk);
  }
  return rs;
}

template <int D>
struct FwdSmem {
  static constexpr int TILE = 128 * D * 2;            // one [128 x D] operand
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = TILE;                  // 2 stages
  static constexpr int OFF_V = 3 * TILE;              // 2 stages
  static constexpr int OFF_BAR = 5 * TILE;            // P never touches shared memory (it lives in TMEM)
  static constexpr int TOTAL = OFF_BAR + 128 + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using L = FwdSmem<D>;
  constexpr int PANELS = D / 64;
  // TMEM columns: S fp32 [0,128); P (bf16 pairs, 64 words per row) overwrites S in place as each
  // thread finishes reading its row; P V product at [128, 128 + D)
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t IDESC_S = umma_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t IDESC_PV = umma_idesc_bf16(128, D, 0, 1);

  int start, len, qb, nblk;
  if (!locate_block(a.cu, a.n_docs, blockIdx.x, start, len, qb, nblk)) return;
  qb = nblk - 1 - qb;                                  // heaviest (most kv blocks) first
  const int h = blockIdx.y;
  const int hkv = h / (a.hq / a.hk);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);   // [2]
  uint64_t* bar_q = kv_full + 2;
  uint64_t* bar_s = kv_full + 3;
  uint64_t* bar_o = kv_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_full + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(kv_full, 1); mbar_init(kv_full + 1, 1);
    mbar_init(bar_q, 1); mbar_init(bar_s, 1); mbar_init(bar_o, 1);
    mbar_fence_init();
    *abort_flag = a.status[0] != 0 ? 1 : 0;
  }
  __syncthreads();
  if (*abort_flag) return;
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_row = tmem + (static_cast<uint32_t>(warp * 32) << 16);

  const int n_kv = qb + 1;
  const int q_row0 = start + qb * 128;
  auto load_kv = [&](int j) {
    const int st = j & 1;
    mbar_expect_tx(kv_full + st, 2 * L::TILE);
#pragma unroll
    for (int p = 0; p < PANELS; ++p) {
      tma_load_2d(sK + st * L::TILE + p * 16384, &tmK, kv_full + st, hkv * D + p * 64, start + j * 128);
      tma_load_2d(sV + st * L::TILE + p * 16384, &tmV, kv_full + st, hkv * D + p * 64, start + j * 128);
    }
  };
  auto issue_s = [&](int j) {
    const uint32_t qa = smem_u32(sQ), kb = smem_u32(sK + (j & 1) * L::TILE);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      umma_f16_ss(tmem, desc_kmajor(qa, kk), desc_kmajor(kb, kk), IDESC_S, kk != 0);
    umma_commit(bar_s);
  };

  bool ok = true;
  if (tid == 0) {
    mbar_expect_tx(bar_q, L::TILE);
#pragma unroll
    for (int p = 0; p < PANELS; ++p) tma_load_2d(sQ + p * 16384, &tmQ, bar_q, h * D + p * 64, q_row0);
    load_kv(0);
    if (n_kv > 1) load_kv(1);
    ok &= mbar_wait(bar_q, 0, abort_flag, a.status, CB_ERR_WAIT_FULL);
    ok &= mbar_wait(kv_full, 0, abort_flag, a.status, CB_ERR_WAIT_FULL);
    if (ok) { tc_fence_after(); issue_s(0); }
  }

  const int r = tid;                                   // my row of the tile
  const float sl2 = a.scale * LOG2E;
  float m_run = -INFINITY, l_run = 0.f;
  float o[D];
#pragma unroll
  for (int i = 0; i < D; ++i) o[i] = 0.f;

  for (int j = 0; j < n_kv; ++j) {
    ok &= mbar_wait(bar_s, j & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    const bool diag = (j == qb);
    // pass 1: row maximum of the raw scores
    const float mx = diag ? fwd_row_max<true>(t_row, r) : fwd_row_max<false>(t_row, r);
    if (j > 0) {
      // previous P V product: fold into the running output before rescaling it
      ok &= mbar_wait(bar_o, (j - 1) & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t pv[32];
        tmem_ld_32x32(t_row + 128 + c * 32, pv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(pv[i]);
      }
      if (tid == 0 && ok && j + 1 < n_kv) load_kv(j + 1);   // stage (j+1)&1 was released by P V of block j-1
    }
    const float m_new = fmaxf(m_run, mx);
    const float alpha = ex2_approx((m_run - m_new) * sl2);
    const float mb = m_new * sl2;
    const float rs = diag ? fwd_row_exp<true>(t_row, r, sl2, mb) : fwd_row_exp<false>(t_row, r, sl2, mb);
    tmem_st_wait();
    l_run = l_run * alpha + rs;
    m_run = m_new;
    if (__any_sync(0xffffffffu, alpha != 1.f)) {     // the row maximum rarely moves after the first blocks
#pragma unroll
      for (int i = 0; i < D; ++i) o[i] *= alpha;
    }
    tc_fence_before();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t vb = smem_u32(sV + (j & 1) * L::TILE);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)      // A = P from TMEM: 16 bf16 of K per step = 8 words
        umma_f16_ts(tmem + 128, tmem + kk * 8, desc_mnmajor(vb, kk), IDESC_PV, kk != 0);
      umma_commit(bar_o);
      if (j + 1 < n_kv) {
        ok &= mbar_wait(kv_full + ((j + 1) & 1), ((j + 1) >> 1) & 1, abort_flag, a.status, CB_ERR_WAIT_FULL);
        if (ok) { tc_fence_after(); issue_s(j + 1); }
      }
    }
  }
  if (ok) {
    ok &= mbar_wait(bar_o, (n_kv - 1) & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t pv[32];
      tmem_ld_32x32(t_row + 128 + c * 32, pv);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(pv[i]);
    }
    const int rg = qb * 128 + r;
    if (ok && rg < len) {
      const float inv = 1.f / l_run;
      const long long t = start + rg;
      CB_DEBUG_CHECK_ST(a.status, t >= 0 && t < a.T, CB_DBG_ATTN_ROW, t);
      uint4* op = reinterpret_cast<uint4*>(a.O + t * a.ldo + static_cast<long long>(h) * D);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        uint4 u;
        u.x = pack_bf16x2(o[8 * c + 0] * inv, o[8 * c + 1] * inv);
        u.y = pack_bf16x2(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
        u.z = pack_bf16x2(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
        u.w = pack_bf16x2(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
        op[c] = u;
      }
      a.lse[static_cast<long long>(h) * a.T + t] = m_run * a.scale + __logf(l_run);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------------
// Forward, second form (opt-in, see cb_attn_fwd): two threads per score row and one pass over S.
// 256 threads: warps w and w + 4 own the same 32 TMEM lanes (score rows) and split the 128 columns of S (and
// the D columns of O) in halves.  Each thread reads its 64 scores once, the two halves of a row exchange their
// maxima through shared memory (a 64-thread named barrier per lane quarter), and the probabilities go back to
// TMEM as bf16 over the S columns both halves have finished reading.  O is never held in registers: the P V
// products accumulate in TMEM across kv blocks, and a warp rescales its slice of O in place only when one of its
// rows saw a larger maximum (rare after the first blocks of a causal row).  Per kv block a thread therefore runs
// 64 instead of 256 score visits and the per-block O read-back disappears.
__device__ __forceinline__ void pair_bar_sync(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

template <int D>
__global__ void __launch_bounds__(BWD2_THREADS, (D == 64 ? 2 : 1))
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using L = FwdSmem<D>;
  constexpr int PANELS = D / 64;
  constexpr int DH = D / 2;                            // O columns per thread
  constexpr uint32_t TMEM_COLS = 256;                  // S / P at [0, 128), O at [128, 128 + D)
  constexpr uint32_t IDESC_S = umma_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t IDESC_PV = umma_idesc_bf16(128, D, 0, 1);

  int start, len, qb, nblk;
  if (!locate_block(a.cu, a.n_docs, blockIdx.x, start, len, qb, nblk)) return;
  qb = nblk - 1 - qb;                                  // heaviest (most kv blocks) first
  const int h = blockIdx.y;
  const int hkv = h / (a.hq / a.hk);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);   // [2]
  uint64_t* bar_q = kv_full + 2;
  uint64_t* bar_s = kv_full + 3;
  uint64_t* bar_o = kv_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(kv_full + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float s_x[2][128];                        // per-row exchange between the two column halves

  const int tid = threadIdx.x, warp = tid >> 5;
  const int q4 = warp & 3, half = warp >> 2;
  if (tid == 0) {
    mbar_init(kv_full, 1); mbar_init(kv_full + 1, 1);
    mbar_init(bar_q, 1); mbar_init(bar_s, 1); mbar_init(bar_o, 1);
    mbar_fence_init();
    *abort_flag = a.status[0] != 0 ? 1 : 0;
  }
  __syncthreads();
  if (*abort_flag) return;
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_row = tmem + (static_cast<uint32_t>(q4 * 32) << 16);

  const int n_kv = qb + 1;
  const int q_row0 = start + qb * 128;
  auto load_kv = [&](int j) {
    const int st = j & 1;
    mbar_expect_tx(kv_full + st, 2 * L::TILE);
#pragma unroll
    for (int p = 0; p < PANELS; ++p) {
      tma_load_2d(sK + st * L::TILE + p * 16384, &tmK, kv_full + st, hkv * D + p * 64, start + j * 128);
      tma_load_2d(sV + st * L::TILE + p * 16384, &tmV, kv_full + st, hkv * D + p * 64, start + j * 128);
    }
  };
  auto issue_s = [&](int j) {
    const uint32_t qa = smem_u32(sQ), kb = smem_u32(sK + (j & 1) * L::TILE);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      umma_f16_ss(tmem, desc_kmajor(qa, kk), desc_kmajor(kb, kk), IDESC_S, kk != 0);
    umma_commit(bar_s);
  };

  bool ok = true;
  if (tid == 0) {
    mbar_expect_tx(bar_q, L::TILE);
#pragma unroll
    for (int p = 0; p < PANELS; ++p) tma_load_2d(sQ + p * 16384, &tmQ, bar_q, h * D + p * 64, q_row0);
    load_kv(0);
    if (n_kv > 1) load_kv(1);
    ok &= mbar_wait(bar_q, 0, abort_flag, a.status, CB_ERR_WAIT_FULL);
    ok &= mbar_wait(kv_full, 0, abort_flag, a.status, CB_ERR_WAIT_FULL);
    if (ok) { tc_fence_after(); issue_s(0); }
  }

  const int r = q4 * 32 + (tid & 31);                  // my row of the tile
  const int c0 = half * 64;                            // my first score column
  const float sl2 = a.scale * LOG2E;
  float m_run = -INFINITY, l_run = 0.f;                // l_run: this half's share of the row sum

  for (int j = 0; j < n_kv; ++j) {
    ok &= mbar_wait(bar_s, j & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    const bool diag = (j == qb);
    uint32_t s[64];
    tmem_ld_32x32(t_row + c0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
    tmem_ld_32x32(t_row + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
    tmem_ld_wait();
    float mx = -INFINITY;
    if (diag) {
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (c0 + i <= r) mx = fmaxf(mx, __uint_as_float(s[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(s[i]));
    }
    s_x[half][r] = mx;
    pair_bar_sync(1 + q4);                             // both halves have read their scores and posted their maxima
    mx = fmaxf(mx, s_x[half ^ 1][r]);
    const float m_new = fmaxf(m_run, mx);
    const float alpha = ex2_approx((m_run - m_new) * sl2);
    const float mb = m_new * sl2;
    float rs = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float e0 = ex2_approx(fmaf(__uint_as_float(s[32 * c + 2 * i]), sl2, -mb));
        float e1 = ex2_approx(fmaf(__uint_as_float(s[32 * c + 2 * i + 1]), sl2, -mb));
        if (diag) {
          e0 = (c0 + 32 * c + 2 * i <= r) ? e0 : 0.f;
          e1 = (c0 + 32 * c + 2 * i + 1 <= r) ? e1 : 0.f;
        }
        rs += e0 + e1;
        pk[i] = pack_bf16x2(e0, e1);
      }
      // bf16 pairs of columns [c0 + 32c, c0 + 32c + 32) -> TMEM words [c0 / 2 + 16c, + 16) of my row
      tmem_st_32x16(t_row + (c0 >> 1) + 16 * c, pk);
    }
    l_run = l_run * alpha + rs;
    m_run = m_new;
    if (j > 0) {
      // the previous P V product has landed in O (and released its K / V stage)
      ok &= mbar_wait(bar_o, (j - 1) & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      if (tid == 0 && ok && j + 1 < n_kv) load_kv(j + 1);
      if (__any_sync(0xffffffffu, alpha != 1.f)) {     // a row of this warp has a new maximum: rescale my slice of O
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(t_row + 128 + half * DH + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(t_row + 128 + half * DH + c * 32, o);
        }
      }
    }
    tmem_st_wait();
    tc_fence_before();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t vb = smem_u32(sV + (j & 1) * L::TILE);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)      // A = P from TMEM: 16 bf16 of K per step = 8 words; O accumulates across blocks
        umma_f16_ts(tmem + 128, tmem + kk * 8, desc_mnmajor(vb, kk), IDESC_PV, (j | kk) != 0);
      umma_commit(bar_o);
      if (j + 1 < n_kv) {
        ok &= mbar_wait(kv_full + ((j + 1) & 1), ((j + 1) >> 1) & 1, abort_flag, a.status, CB_ERR_WAIT_FULL);
        if (ok) { tc_fence_after(); issue_s(j + 1); }
      }
    }
  }
  if (ok) ok &= mbar_wait(bar_o, (n_kv - 1) & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
  s_x[half][r] = l_run;
  pair_bar_sync(1 + q4);                                 // reached by every thread, whatever its waits returned
  if (ok) {
    tc_fence_after();
    const float l_tot = l_run + s_x[half ^ 1][r];
    const int rg = qb * 128 + r;
    const bool row_ok = ok && rg < len;
    const float inv = 1.f / l_tot;
    const long long t = start + rg;
#pragma unroll
    for (int c = 0; c < DH / 32; ++c) {
      uint32_t o[32];
      tmem_ld_32x32(t_row + 128 + half * DH + c * 32, o);
      tmem_ld_wait();
      if (row_ok) {
        uint4* op = reinterpret_cast<uint4*>(a.O + t * a.ldo + static_cast<long long>(h) * D + half * DH + c * 32);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(o[8 * k + 0]) * inv, __uint_as_float(o[8 * k + 1]) * inv);
          u.y = pack_bf16x2(__uint_as_float(o[8 * k + 2]) * inv, __uint_as_float(o[8 * k + 3]) * inv);
          u.z = pack_bf16x2(__uint_as_float(o[8 * k + 4]) * inv, __uint_as_float(o[8 * k + 5]) * inv);
          u.w = pack_bf16x2(__uint_as_float(o[8 * k + 6]) * inv, __uint_as_float(o[8 * k + 7]) * inv);
          op[k] = u;
        }
      }
    }
    if (row_ok && half == 0) a.lse[static_cast<long long>(h) * a.T + t] = m_run * a.scale + __logf(l_tot);
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d].  LANES = D / 8 lanes share one (t, h): each loads 16 bytes
// of dO and of O, so a warp reads 512 contiguous bytes of each tensor per instruction (32 / LANES heads of
// one token, or of neighbouring tokens when the rows are dense) and the sum needs log2(LANES) shuffles.
template <int LANES>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const bf16* __restrict__ dO, const bf16* __restrict__ O, long long ld_do, long long ld_o, int T,
                  int hq, float* __restrict__ delta) {
  constexpr int D = LANES * 8;
  const long long gid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long pair = gid / LANES;                       // (t, h) index, h fastest
  const int sub = static_cast<int>(gid % LANES);
  const bool in = pair < static_cast<long long>(T) * hq;
  float s = 0.f;
  long long t = 0;
  int h = 0;
  if (in) {
    t = pair / hq;
    h = static_cast<int>(pair - t * hq);
    const uint4 a = *reinterpret_cast<const uint4*>(dO + t * ld_do + static_cast<long long>(h) * D + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(O + t * ld_o + static_cast<long long>(h) * D + sub * 8);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
    s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (in && sub == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// the same sum for head sizes the vector kernel does not cover: one warp per (t, h)
__global__ void attn_delta_generic_kernel(const bf16* __restrict__ dO, const bf16* __restrict__ O, long long ld_do,
                                          long long ld_o, int T, int hq, int D, float* __restrict__ delta) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(T) * hq) return;
  const long long t = w / hq;
  const int h = static_cast<int>(w % hq);
  const bf16* a = dO + t * ld_do + static_cast<long long>(h) * D;
  const bf16* b = O + t * ld_o + static_cast<long long>(h) * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + i));
    const float2 y = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(b + i));
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

}  // namespace cb

// =========================================================================================== backward
namespace cb {

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ---------------------------------------------------------------------------------------------------
// Backward.  One CTA: kv block `jb` of one document, one query head; loops over the query blocks i >= jb.
// For D = 64 it needs 256 TMEM columns and ~97 KB of shared memory, so two CTAs share an SM and one computes
// its softmax while the other has the tensor core (D = 128: 512 columns, 160 KB, one CTA per SM).
// The S, dP and dQ tiles take turns in the same 128 TMEM columns, and P and dS take turns in one shared
// tile, which turns an iteration into three MMA phases:
//   S = Q K^T            -> P = exp(S - lse)            (P to smem)
//   dV += P^T dO ; dP = dO V^T  -> dS = P (dP - delta)  (P re-read from smem as bf16, dS overwrites it)
//   dK += dS^T Q ; dQ = dS K    -> dQ added to global
// dK / dV are added into [T, hk, D] fp32 accumulators with red.global.add (the query heads of a group are
// different CTAs).
template <int D>
struct Bwd2Smem {
  static constexpr int TILE = 128 * D * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;
  static constexpr int OFF_DO = 3 * TILE;
  static constexpr int OFF_P = 4 * TILE;              // P, then dS (bf16 [128 x 128] operand image)
  static constexpr int OFF_BAR = OFF_P + 32768;
  static constexpr int TOTAL = OFF_BAR + 128 + 1024;
};

// read back 32 consecutive bf16 values of thread-row r from the image written by store_row_chunk32
__device__ __forceinline__ void load_row_chunk32(const uint8_t* base, int r, int c32, float (&v)[32]) {
  const int panel = c32 >> 1;
  const uint8_t* row = base + panel * 16384 + r * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int cc = (c32 & 1) * 4 + q;
    const uint4 u = *reinterpret_cast<const uint4*>(row + ((cc ^ (r & 7)) << 4));
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    v[8 * q + 0] = a.x; v[8 * q + 1] = a.y; v[8 * q + 2] = b.x; v[8 * q + 3] = b.y;
    v[8 * q + 4] = c.x; v[8 * q + 5] = c.y; v[8 * q + 6] = d.x; v[8 * q + 7] = d.y;
  }
}

template <int D>
__global__ void __launch_bounds__(BWD2_THREADS, 2)
attn_bwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmdQ, const AttnArgs a) {
  using L = Bwd2Smem<D>;
  constexpr int PANELS = D / 64;
  constexpr uint32_t TMEM_COLS = (128 + 2 * D) <= 256 ? 256 : 512;
  constexpr uint32_t C_S = 0, C_DV = 128, C_DK = 128 + D;                // S, dP and dQ share the first 128 columns
  constexpr uint32_t IDESC_S = umma_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t IDESC_T = umma_idesc_bf16(128, D, 1, 1);            // P^T dO, dS^T Q
  constexpr uint32_t IDESC_DQ = umma_idesc_bf16(128, D, 0, 1);           // dS K

  int start, len, jb, nblk;
  if (!locate_block(a.cu, a.n_docs, blockIdx.x, start, len, jb, nblk)) return;   // jb = 0 is the heaviest
  const int h = blockIdx.y;
  const int hkv = h / (a.hq / a.hk);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sdO = smem + L::OFF_DO;
  uint8_t* sP = smem + L::OFF_P;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* bar_kv = q_full + 1;
  uint64_t* bar_s = q_full + 2;
  uint64_t* bar_dp = q_full + 3;
  uint64_t* bar_dq = q_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // 8 warps: warps w and w + 4 own the same 32 TMEM lanes (score rows) and split the columns in halves,
  // which doubles the number of warps available to hide TMEM / shared-memory latency
  const int tid = threadIdx.x, warp = tid >> 5;
  const int q4 = warp & 3, half = warp >> 2;
  if (tid == 0) {
    mbar_init(q_full, 1); mbar_init(bar_kv, 1); mbar_init(bar_s, 1); mbar_init(bar_dp, 1); mbar_init(bar_dq, 1);
    mbar_fence_init();
    *abort_flag = a.status[0] != 0 ? 1 : 0;
  }
  __syncthreads();
  if (*abort_flag) return;
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_row = tmem + (static_cast<uint32_t>(q4 * 32) << 16);

  const int kv_row0 = start + jb * 128;
  const int n_it = nblk - jb;
  auto load_q = [&](int it) {
    const int row0 = start + (jb + it) * 128;
    mbar_expect_tx(q_full, 2 * L::TILE);
#pragma unroll
    for (int p = 0; p < PANELS; ++p) {
      tma_load_2d(sQ + p * 16384, &tmQ, q_full, h * D + p * 64, row0);
      tma_load_2d(sdO + p * 16384, &tmdO, q_full, h * D + p * 64, row0);
    }
  };

  bool ok = true;
  if (tid == 0) {
    mbar_expect_tx(bar_kv, 2 * L::TILE);
#pragma unroll
    for (int p = 0; p < PANELS; ++p) {
      tma_load_2d(sK + p * 16384, &tmK, bar_kv, hkv * D + p * 64, kv_row0);
      tma_load_2d(sV + p * 16384, &tmV, bar_kv, hkv * D + p * 64, kv_row0);
    }
    load_q(0);
    ok &= mbar_wait(bar_kv, 0, abort_flag, a.status, CB_ERR_WAIT_FULL);
  }

  const int r = q4 * 32 + (tid & 31);
  const float sl2 = a.scale * LOG2E;
  const uint32_t kA = smem_u32(sK), vA = smem_u32(sV), pA = smem_u32(sP), qA = smem_u32(sQ), doA = smem_u32(sdO);

  for (int it = 0; it < n_it; ++it) {
    const int i = jb + it;
    if (tid == 0) {
      if (D == 64) tma_store_wait_read<0>();          // the dQ tile of the last iteration has left the P / dS buffer
      ok &= mbar_wait(q_full, it & 1, abort_flag, a.status, CB_ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(tmem + C_S, desc_kmajor(qA, kk), desc_kmajor(kA, kk), IDESC_S, kk != 0);
        umma_commit(bar_s);
      }
    }
    const int rg = i * 128 + r;                      // my query row within the document
    const bool row_ok = rg < len;
    const long long tq = start + rg;
    const float lse2 = row_ok ? a.lse[static_cast<long long>(h) * a.T + tq] * LOG2E : 0.f;
    const float dlt = row_ok ? a.delta[static_cast<long long>(h) * a.T + tq] : 0.f;
    const bool diag = (it == 0);
    // ---- phase 1: P = exp(S - lse), masked, to shared memory
    ok &= mbar_wait(bar_s, it & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
#pragma unroll 1
    for (int c = half * 2; c < half * 2 + 2; ++c) {
      uint32_t s[32];
      float p[32];
      tmem_ld_32x32(t_row + C_S + c * 32, s);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const bool keep = row_ok && (!diag || c * 32 + k <= r);
        const float e = ex2_approx(fmaf(__uint_as_float(s[k]), sl2, -lse2));
        p[k] = keep ? e : 0.f;
      }
      store_row_chunk32(sP, r, c, p);
    }
    tc_fence_before();
    fence_async_smem();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)                  // dV += P^T dO     (K = the 128 query rows)
        umma_f16_ss(tmem + C_DV, desc_mnmajor(pA, kk), desc_mnmajor(doA, kk), IDESC_T, (it | kk) != 0);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)             // dP = dO V^T      (over the columns S occupied)
        umma_f16_ss(tmem + C_S, desc_kmajor(doA, kk), desc_kmajor(vA, kk), IDESC_S, kk != 0);
      umma_commit(bar_dp);
    }
    // ---- phase 2: dS = P (dP - delta) scale, overwriting P in shared memory
    ok &= mbar_wait(bar_dp, it & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
#pragma unroll 1
    for (int c = half * 2; c < half * 2 + 2; ++c) {
      uint32_t dp[32];
      float p[32];
      tmem_ld_32x32(t_row + C_S + c * 32, dp);
      load_row_chunk32(sP, r, c, p);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 32; ++k) p[k] = p[k] * (__uint_as_float(dp[k]) - dlt) * a.scale;
      store_row_chunk32(sP, r, c, p);
    }
    tc_fence_before();
    fence_async_smem();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)                  // dK += dS^T Q
        umma_f16_ss(tmem + C_DK, desc_mnmajor(pA, kk), desc_mnmajor(qA, kk), IDESC_T, (it | kk) != 0);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)                  // dQ = dS K        (K = the 128 kv rows)
        umma_f16_ss(tmem + C_S, desc_kmajor(pA, kk), desc_mnmajor(kA, kk), IDESC_DQ, kk != 0);
      umma_commit(bar_dq);
    }
    // ---- phase 3: dQ out
    ok &= mbar_wait(bar_dq, it & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    if (tid == 0 && ok && it + 1 < n_it) load_q(it + 1);                // Q / dO of this iteration are consumed
    if (D == 64) {
      // dQ tile (fp32) -> the P / dS buffer, which nobody reads any more, as two [128 x 32] boxes in the layout
      // of the dq_acc tensor map -> one TMA reduce-add per box instead of eight red.global.add per thread.
      // Rows past the end of the document carry exact zeros (their P was masked), rows past T are clipped.
      uint32_t dq[32];
      tmem_ld_32x32(t_row + C_S + half * 32, dq);
      tmem_ld_wait();
      uint8_t* dstrow = sP + half * 16384 + r * 128;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc)
        *reinterpret_cast<uint4*>(dstrow + ((cc ^ (r & 7)) << 4)) = make_uint4(dq[4 * cc], dq[4 * cc + 1], dq[4 * cc + 2], dq[4 * cc + 3]);
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(!ok)) { ok = false; break; }
      if (tid == 0) {
        CB_DEBUG_CHECK_ST(a.status, start + i * 128 >= 0 && ((h * D) * 4) % 16 == 0, CB_DBG_TMA_COORD, start + i * 128);
        tma_reduce_add_2d(&tmdQ, sP, h * D, start + i * 128);
        tma_reduce_add_2d(&tmdQ, sP + 16384, h * D + 32, start + i * 128);
        tma_store_commit();
      }
    } else {
#pragma unroll
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t dq[32];
        tmem_ld_32x32(t_row + C_S + c * 32, dq);
        tmem_ld_wait();
        if (row_ok && ok) {
          float* dst = a.dq_acc + (tq * a.hq + h) * D + c * 32;
#pragma unroll
          for (int k = 0; k < 32; k += 4)
            red_add_v4(dst + k, __uint_as_float(dq[k]), __uint_as_float(dq[k + 1]), __uint_as_float(dq[k + 2]),
                       __uint_as_float(dq[k + 3]));
        }
      }
      tc_fence_before();
      if (__syncthreads_or(!ok)) { ok = false; break; }
    }
  }
  if (D == 64 && tid == 0) tma_store_wait_all();
  if (ok) {
    tc_fence_after();
    const int kg = jb * 128 + r;                      // my kv row within the document
    const bool kv_ok = kg < len;
    const long long tk = start + kg;
#pragma unroll
    for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
      uint32_t dv[32], dk[32];
      tmem_ld_32x32(t_row + C_DV + c * 32, dv);
      tmem_ld_32x32(t_row + C_DK + c * 32, dk);
      tmem_ld_wait();
      if (kv_ok) {
        float* pv = a.dv_part + (tk * a.hk + hkv) * D + c * 32;
        float* pk = a.dk_part + (tk * a.hk + hkv) * D + c * 32;
#pragma unroll
        for (int k = 0; k < 32; k += 4) {
          red_add_v4(pv + k, __uint_as_float(dv[k]), __uint_as_float(dv[k + 1]), __uint_as_float(dv[k + 2]),
                     __uint_as_float(dv[k + 3]));
          red_add_v4(pk + k, __uint_as_float(dk[k]), __uint_as_float(dk[k + 1]), __uint_as_float(dk[k + 2]),
                     __uint_as_float(dk[k + 3]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// dqkv[t] = bf16( dQ | sum over the query heads of a group of dK | same for dV ); one block per token,
// four consecutive columns per thread (D is a multiple of 4, so a group never straddles heads)
__global__ void attn_bwd_finalize_kernel(const float* __restrict__ dq_acc, const float* __restrict__ dk_part,
                                         const float* __restrict__ dv_part, bf16* __restrict__ dqkv, long long ld,
                                         int T, int hq, int hk, int D, const int* __restrict__ cu, int n_docs,
                                         int part_heads) {
  // part_heads: heads per token in dk_part / dv_part — hq (one partial per query head, summed here) or hk
  // (already accumulated per kv head by the kernel)
  const long long t = blockIdx.x;
  const int nq = hq * D, nk = hk * D, g = part_heads / hk;
  bf16* out = dqkv + t * ld;
  const bool valid = t < cu[n_docs];                  // padding tokens get zero gradients
  for (int c = threadIdx.x * 4; c < nq + 2 * nk; c += blockDim.x * 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
      if (c < nq) {
        v = *reinterpret_cast<const float4*>(dq_acc + t * nq + c);
      } else {
        const int cc = (c - nq) % nk, which = (c - nq) / nk;
        const int kvh = cc / D, d = cc % D;
        const float* src = (which == 0 ? dk_part : dv_part) + (t * part_heads + static_cast<long long>(kvh) * g) * D + d;
        for (int i = 0; i < g; ++i) {
          const float4 x = *reinterpret_cast<const float4*>(src + static_cast<long long>(i) * D);
          v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
        }
      }
    }
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(out + c) = o;
  }
}

}  // namespace cb

// =========================================================================================== host side
#include "host_common.h"

namespace {

int attn_maps(CUtensorMap* mq, CUtensorMap* mk, CUtensorMap* mv, const void* q, const void* k, const void* v, int T,
              int hq, int hk, int D, long long ldq, long long ldk, long long ldv) {
  int e = cbhost::make_tmap(mq, q, static_cast<unsigned long long>(hq) * D, T, ldq, 64, 128);
  if (e) return e;
  e = cbhost::make_tmap(mk, k, static_cast<unsigned long long>(hk) * D, T, ldk, 64, 128);
  if (e) return e;
  return cbhost::make_tmap(mv, v, static_cast<unsigned long long>(hk) * D, T, ldv, 64, 128);
}

template <typename K>
int set_smem(K kern, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace

extern "C" {

// q [T, hq, D] (row pitch ldq elements), k / v [T, hk, D]; cu: int32 [n_docs + 1] on the device.
// o [T, hq, D] with pitch ldo; lse [hq, T] fp32.  Rows at or beyond cu[n_docs] are left untouched
// (the caller zero-fills o).  D is 64 or 128, hq a multiple of hk.
int cb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu, int n_docs, int T,
                int hq, int hk, int D, long long ldq, long long ldk, long long ldv, long long ldo, float scale,
                int* status, void* stream) {
  if ((D != 64 && D != 128) || hq % hk != 0 || T <= 0 || n_docs <= 0) return -1;
  CUtensorMap mq, mk, mv;
  int e = attn_maps(&mq, &mk, &mv, q, k, v, T, hq, hk, D, ldq, ldk, ldv);
  if (e) return e;
  cb::AttnArgs a = {};
  a.T = T; a.hq = hq; a.hk = hk; a.n_docs = n_docs; a.cu = cu; a.scale = scale;
  a.O = static_cast<cb::bf16*>(o); a.ldo = ldo; a.lse = lse; a.status = status;
  dim3 grid((T + 127) / 128 + n_docs, hq);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // CB_ATTN_FWD=2 in the environment selects the two-threads-per-row kernel.  Measured on the 0.5B shape
  // (8 x 1024 tokens, 14 heads): 68.7 us against 61.0 us for the one-thread-per-row kernel below, which therefore
  // stays the default: a kv block costs a chain of dependent hops (MMA commit -> TMEM load -> exchange -> TMEM
  // store -> CTA barrier -> MMA), and halving the arithmetic per thread does not shorten that chain.
  static const bool two_thread_rows = [] { const char* v = getenv("CB_ATTN_FWD"); return v != nullptr && v[0] == '2'; }();
  if (two_thread_rows) {
    if (D == 64) {
      static bool cfg = false;
      if (!cfg) { e = set_smem(cb::attn_fwd2_kernel<64>, cb::FwdSmem<64>::TOTAL); if (e) return e; cfg = true; }
      cb::attn_fwd2_kernel<64><<<grid, cb::BWD2_THREADS, cb::FwdSmem<64>::TOTAL, s>>>(mq, mk, mv, a);
    } else {
      static bool cfg = false;
      if (!cfg) { e = set_smem(cb::attn_fwd2_kernel<128>, cb::FwdSmem<128>::TOTAL); if (e) return e; cfg = true; }
      cb::attn_fwd2_kernel<128><<<grid, cb::BWD2_THREADS, cb::FwdSmem<128>::TOTAL, s>>>(mq, mk, mv, a);
    }
    return static_cast<int>(cudaGetLastError());
  }
  if (D == 64) {
    static bool cfg = false;
    if (!cfg) { e = set_smem(cb::attn_fwd_kernel<64>, cb::FwdSmem<64>::TOTAL); if (e) return e; cfg = true; }
    cb::attn_fwd_kernel<64><<<grid, cb::ATT_THREADS, cb::FwdSmem<64>::TOTAL, s>>>(mq, mk, mv, a);
  } else {
    static bool cfg = false;
    if (!cfg) { e = set_smem(cb::attn_fwd_kernel<128>, cb::FwdSmem<128>::TOTAL); if (e) return e; cfg = true; }
    cb::attn_fwd_kernel<128><<<grid, cb::ATT_THREADS, cb::FwdSmem<128>::TOTAL, s>>>(mq, mk, mv, a);
  }
  return static_cast<int>(cudaGetLastError());
}

// Backward.  scratch: delta [hq*T] fp32, dq_acc [T*hq*D] fp32, dk_part / dv_part [T*hk*D] fp32 (all three
// accumulators are zeroed here).  dqkv: bf16 [T, (hq + 2 hk) * D] with row pitch ld_dqkv receives dQ | dK | dV.
int cb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                const int* cu, int n_docs, int T, int hq, int hk, int D, long long ldq, long long ldk, long long ldv,
                long long ldo, long long ld_do, float scale, float* delta, float* dq_acc, float* dk_part,
                float* dv_part, void* dqkv, long long ld_dqkv, int* status, void* stream) {
  if ((D != 64 && D != 128) || hq % hk != 0 || T <= 0 || n_docs <= 0) return -1;
  CUtensorMap mq, mk, mv, mdo;
  int e = attn_maps(&mq, &mk, &mv, q, k, v, T, hq, hk, D, ldq, ldk, ldv);
  if (e) return e;
  e = cbhost::make_tmap(&mdo, d_o, static_cast<unsigned long long>(hq) * D, T, ld_do, 64, 128);
  if (e) return e;
  CUtensorMap mdq;                                      // fp32 dQ accumulator [T, hq * D], boxes of 128 rows x 32 columns
  e = cbhost::make_tmap(&mdq, dq_acc, static_cast<unsigned long long>(hq) * D, T, static_cast<unsigned long long>(hq) * D,
                        32, 128, 4);
  if (e) return e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long pairs = static_cast<long long>(T) * hq;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(d_o) & 15) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0 &&
                      ld_do % 8 == 0 && ldo % 8 == 0;
  if (vec_ok && D == 64) {
    cb::attn_delta_kernel<8><<<static_cast<unsigned>((pairs * 8 + 255) / 256), 256, 0, s>>>(
        static_cast<const cb::bf16*>(d_o), static_cast<const cb::bf16*>(o), ld_do, ldo, T, hq, delta);
  } else if (vec_ok && D == 128) {
    cb::attn_delta_kernel<16><<<static_cast<unsigned>((pairs * 16 + 255) / 256), 256, 0, s>>>(
        static_cast<const cb::bf16*>(d_o), static_cast<const cb::bf16*>(o), ld_do, ldo, T, hq, delta);
  } else {
    cb::attn_delta_generic_kernel<<<static_cast<unsigned>((pairs * 32 + 255) / 256), 256, 0, s>>>(
        static_cast<const cb::bf16*>(d_o), static_cast<const cb::bf16*>(o), ld_do, ldo, T, hq, D, delta);
  }
  CB_CHECK_CUDA(cudaMemsetAsync(dq_acc, 0, sizeof(float) * static_cast<size_t>(T) * hq * D, s));
  cb::AttnArgs a = {};
  a.T = T; a.hq = hq; a.hk = hk; a.n_docs = n_docs; a.cu = cu; a.scale = scale;
  a.lse = const_cast<float*>(lse); a.delta = delta; a.dq_acc = dq_acc; a.dk_part = dk_part; a.dv_part = dv_part;
  a.status = status;
  dim3 grid((T + 127) / 128 + n_docs, hq);
  // Two threads per score row, S / dP / dQ sharing TMEM columns, dK / dV accumulated per kv head with red.add
  // (so those buffers start from zero).  D = 64 additionally fits two CTAs per SM.
  const int part_heads = hk;
  CB_CHECK_CUDA(cudaMemsetAsync(dk_part, 0, sizeof(float) * static_cast<size_t>(T) * hk * D, s));
  CB_CHECK_CUDA(cudaMemsetAsync(dv_part, 0, sizeof(float) * static_cast<size_t>(T) * hk * D, s));
  if (D == 64) {
    static bool cfg = false;
    if (!cfg) { e = set_smem(cb::attn_bwd2_kernel<64>, cb::Bwd2Smem<64>::TOTAL); if (e) return e; cfg = true; }
    cb::attn_bwd2_kernel<64><<<grid, cb::BWD2_THREADS, cb::Bwd2Smem<64>::TOTAL, s>>>(mq, mk, mv, mdo, mdq, a);
  } else {
    static bool cfg = false;
    if (!cfg) { e = set_smem(cb::attn_bwd2_kernel<128>, cb::Bwd2Smem<128>::TOTAL); if (e) return e; cfg = true; }
    cb::attn_bwd2_kernel<128><<<grid, cb::BWD2_THREADS, cb::Bwd2Smem<128>::TOTAL, s>>>(mq, mk, mv, mdo, mdq, a);
  }
  cb::attn_bwd_finalize_kernel<<<T, 128, 0, s>>>(dq_acc, dk_part, dv_part, static_cast<cb::bf16*>(dqkv), ld_dqkv, T,
                                                  hq, hk, D, cu, n_docs, part_heads);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
