// Varlen causal GQA flash attention, forward and backward, on tcgen05 tensor
// cores with the score tiles in TMEM.
//
// Layout: q [T, hq, D], k/v [T, hk, D] packed tokens (any row pitch, so they may
// be slices of one fused QKV buffer); documents are the intervals of
// cu_seqlens.  A tile is one 128-row block of one document and one query head;
// tiles are handed out by descending weight over all documents (locate_tile).
//
//   forward : S = Q K^T -> P = softmax -> O += P V        (2 MMAs per kv block)
//   backward: S, dP = dO V^T -> P, dS -> dV += P^T dO, dK += dS^T Q, dQ = dS K
//
// Forward kernels: attn_fwd3_kernel (default: 64-row kv blocks, double-buffered
// S, O accumulated in TMEM, P consumed from TMEM, dedicated MMA and TMA warps, one
// thread per score row, no CTA barrier in the loop); attn_fwd_kernel (first form:
// 128-row kv blocks, O in registers) and attn_fwd2_kernel (two threads per row)
// are kept for comparison (CB_ATTN_FWD=1 / 2).  Backward: attn_bwd2_kernel (one
// CTA per kv block and head, two threads per score row, S / dP / dQ sharing TMEM
// columns, dQ out by TMA reduce-add) with attn_delta_kernel before and
// attn_bwd_finalize_kernel after it.
//
// Every thread that owns a score row reads it from TMEM with tcgen05.ld, so the
// softmax needs no cross-thread shuffles.  The same swizzled image of a [128 x 64]
// bf16 tile serves as a K-major operand (rows = M/N) and as an MN-major operand
// (rows = K), so P^T and dS^T need no transposed copy.  All tensor maps cover this
// GPU's own memory only.
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
  int o_tma;            // forward: a tensor map over O exists, whole blocks may leave by TMA store
};

// Phase timers (compiled in with -DCB_ATTN_PHASE_TIMERS only): two threads of every CTA - the MMA-issuing thread
// and one thread of another warp - add the SM clock cycles they spend between consecutive marks to a global
// table, which cb_attn_phase_read() copies out.  The default build contains none of this.
#ifdef CB_ATTN_PHASE_TIMERS
__device__ unsigned long long cb_attn_phase[2][16];
#define CB_PHASE_DECL_T(ta, tb) const int ph_who = (threadIdx.x == (ta)) ? 0 : ((threadIdx.x == (tb)) ? 1 : -1); \
                      long long ph_t = clock64(); unsigned long long ph_acc[13] = {}
#define CB_PHASE(n) do { if (ph_who >= 0) { const long long t_ = clock64(); ph_acc[n] += t_ - ph_t; ph_t = t_; } } while (0)
#define CB_PHASE_FLUSH do { if (ph_who >= 0) { for (int i_ = 0; i_ < 13; ++i_) atomicAdd(&cb_attn_phase[ph_who][i_], ph_acc[i_]); \
                                               atomicAdd(&cb_attn_phase[ph_who][15], 1ull); } } while (0)
#define CB_PHASE_DECL CB_PHASE_DECL_T(0, 96)
#else
#define CB_PHASE_DECL
#define CB_PHASE_DECL_T(ta, tb)
#define CB_PHASE(n)
#define CB_PHASE_FLUSH
#endif

// Which tile a CTA owns.  A tile is one 128-row block of one document; its weight is the number of 128-row
// blocks its main loop visits (forward: kv blocks up to the diagonal; backward: query blocks from the diagonal
// on), so a document of nb blocks has exactly one tile of every weight 1..nb.  Tiles are handed out by
// descending weight over ALL documents (ties in document order): the heaviest tiles of the batch start first and
// the last wave consists of single-block tiles, whatever the mix of document lengths.  Every warp runs this by
// itself with warp-wide votes (no shared memory, so it can precede the CTA's set-up); cost is one pass over the
// document lengths per weight level.
__device__ __forceinline__ bool locate_tile(const int* cu, int n_docs, int b, int& start, int& len, int& weight, int& nblk,
                                            int* beyond = nullptr) {
  const int lane = threadIdx.x & 31;
  int maxnb = 0;
  for (int d = lane; d < n_docs; d += 32) maxnb = max(maxnb, (cu[d + 1] - cu[d] + 127) >> 7);
  maxnb = __reduce_max_sync(0xffffffffu, maxnb);
  for (int L = maxnb; L >= 1; --L) {
    int cnt = 0;
    for (int d = lane; d < n_docs; d += 32) cnt += (((cu[d + 1] - cu[d] + 127) >> 7) >= L) ? 1 : 0;
    const int tot = __reduce_add_sync(0xffffffffu, cnt);
    if (b < tot) {
      for (int d0 = 0; d0 < n_docs; d0 += 32) {        // the b-th document, in document order, with >= L blocks
        const int d = d0 + lane;
        const bool has = d < n_docs && (((cu[d + 1] - cu[d] + 127) >> 7) >= L);
        const unsigned m = __ballot_sync(0xffffffffu, has);
        const int c = __popc(m);
        if (b < c) {
          const int pos = d0 + __fns(m, 0, b + 1);
          start = cu[pos]; len = cu[pos + 1] - start; nblk = (len + 127) >> 7; weight = L;
          return true;
        }
        b -= c;
      }
      return false;
    }
    b -= tot;
  }
  if (beyond != nullptr) *beyond = b;                  // index among the CTAs past the last tile
  return false;
}

// The grid holds at least ceil((T - cu[n_docs]) / 128) CTAs past the last tile (per head).  In the forward
// kernels they write the zeros of the padding rows at or after cu[n_docs], 128 rows x D columns each, so the
// caller need not clear the output first.
template <int D>
__device__ __forceinline__ void zero_padding_rows(const AttnArgs& a, int beyond, int h) {
  const int valid = a.cu[a.n_docs];
  const long long row0 = static_cast<long long>(valid) + static_cast<long long>(beyond) * 128;
  constexpr int CH = D / 8;                            // 16-byte chunks per row of one head
  for (int i = threadIdx.x; i < 128 * CH; i += blockDim.x) {
    const long long t = row0 + i / CH;
    if (t < a.T) reinterpret_cast<uint4*>(a.O + t * a.ldo + static_cast<long long>(h) * D)[i % CH] = make_uint4(0u, 0u, 0u, 0u);
  }
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

// the same for 32 values already packed as bf16 pairs
__device__ __forceinline__ void store_row_chunk32_packed(uint8_t* base, int r, int c32, const uint32_t (&v)[16]) {
  const int panel = c32 >> 1;
  uint8_t* row = base + panel * 16384 + r * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int cc = (c32 & 1) * 4 + q;
    *reinterpret_cast<uint4*>(row + ((cc ^ (r & 7)) << 4)) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
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
  int beyond = 0;
  if (!locate_tile(a.cu, a.n_docs, blockIdx.y, start, len, qb, nblk, &beyond)) {
    zero_padding_rows<D>(a, beyond, blockIdx.x);
    return;
  }
  qb -= 1;                                             // weight = kv blocks up to the diagonal = qb + 1
  const int h = blockIdx.x;
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
  int beyond = 0;
  if (!locate_tile(a.cu, a.n_docs, blockIdx.y, start, len, qb, nblk, &beyond)) {
    zero_padding_rows<D>(a, beyond, blockIdx.x);
    return;
  }
  qb -= 1;                                             // weight = kv blocks up to the diagonal = qb + 1
  const int h = blockIdx.x;
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


// ---------------------------------------------------------------------------------------------------
// Forward, pipelined form (the default, see cb_attn_fwd).
//
// The two forms above run S-MMA -> softmax -> PV-MMA -> S-MMA of one CTA strictly one after the other and rely on
// a second resident CTA to fill the gaps.  Here the tensor core works in the shadow of the softmax inside ONE CTA:
//   * kv blocks are 64 rows, so a score tile [128 x 64] fp32 takes 64 TMEM columns and two of them plus the
//     output accumulator [128 x D] fit in 256 columns for D = 64 and D = 128 alike (two CTAs per SM);
//   * S(j+1) is computed while the softmax threads work on S(j) (the scores are double-buffered); P(j) (bf16)
//     overwrites the first 32 columns of S(j) and is consumed from TMEM by the P V product, which accumulates O in
//     TMEM over the whole kv loop, so the output never travels through registers inside the loop;
//   * a fifth warp issues every MMA and a sixth owns the TMA rings (K and V blocks, separate rings, stages handed
//     back by tcgen05.commit); the four softmax warps
//     never meet at a CTA barrier: they signal "P(j) written, S(j) consumed" on an mbarrier and move straight on to
//     S(j+1), which is already complete in the other buffer;
//   * one pass over the scores: a thread keeps its 64 scores of the block in registers, takes their maximum, and
//     exponentiates against a reference maximum that is only raised when the block's maximum exceeds it by more
//     than 2^8 (the probabilities then stay below 256, exact in fp32 sums and harmless in bf16); raising it
//     rescales the thread's own O row in TMEM, which after the first blocks of a causal row is rare.
// Per kv block a softmax thread issues about 64 x (max, fma, ex2, add, half a cvt) instructions and nothing else;
// the exp2 unit (16 results per clock and SM) is the bound: 1024 cycles per [128 x 128] of scores.
constexpr int FWD3_THREADS = 192;                      // 4 softmax warps + the MMA-issuing warp + the TMA warp
constexpr float FWD3_RAISE_LOG2 = 8.f;                 // raise the reference maximum only beyond 2^8

template <int D>
struct Fwd3Smem {
  static constexpr int NS = (D == 64) ? 4 : 2;         // depth of the K ring and of the V ring (64-row blocks)
  static constexpr int QT = 128 * D * 2;               // Q tile [128 x D]: D/64 panels of 16 KB
  static constexpr int KT = 64 * D * 2;                // one K or V block [64 x D]: D/64 panels of 8 KB
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = QT;
  static constexpr int OFF_V = QT + NS * KT;
  static constexpr int OFF_BAR = QT + 2 * NS * KT;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(FWD3_THREADS, 2)
attn_fwd3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const AttnArgs a) {
  using L = Fwd3Smem<D>;
  constexpr int NS = L::NS;
  constexpr int PANELS = D / 64;
  constexpr uint32_t TMEM_COLS = 256;                  // S0 [0, 64)  S1 [64, 128)  O [128, 128 + D)
  constexpr uint32_t C_O = 128;
  // D = 64 leaves 64 columns: P(j) goes to its own 32 columns (P0 [192, 224), P1 [224, 256)) instead of over S(j),
  // so S(j+2) may overwrite S(j) as soon as the softmax threads hold the scores in registers - a whole
  // exponentiation pass earlier than "P(j) written".  D = 128 fills all 256 columns and keeps P over S.
  constexpr bool P_APART = (D == 64);
  constexpr uint32_t C_P = 192;
  constexpr uint32_t IDESC_S = umma_idesc_bf16(128, 64, 0, 0);
  constexpr uint32_t IDESC_PV = umma_idesc_bf16(128, D, 0, 1);

  int start, len, qb, nblk;
  int beyond = 0;
  if (!locate_tile(a.cu, a.n_docs, blockIdx.y, start, len, qb, nblk, &beyond)) {
    zero_padding_rows<D>(a, beyond, blockIdx.x);
    return;
  }
  qb -= 1;
  const int h = blockIdx.x;
  const int hkv = h / (a.hq / a.hk);
  const int n_kv = min(2 * qb + 2, (len + 63) >> 6);   // 64-row kv blocks up to and including the diagonal

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint64_t* k_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);    // [NS]
  uint64_t* v_full = k_full + NS;                                       // [NS]
  uint64_t* k_empty = v_full + NS;                                      // [NS] S of the stage's block complete
  uint64_t* v_empty = k_empty + NS;                                     // [NS] P V of the stage's block complete
  uint64_t* bar_s = v_empty + NS;                                       // [2]  S(j) complete in buffer j & 1
  uint64_t* p_ready = bar_s + 2;                                        // [2]  128 arrivals: P(j) written, S(j) consumed
  uint64_t* bar_o = p_ready + 2;                                        //      P V product of block j complete (phase j)
  uint64_t* bar_q = bar_o + 1;
  uint64_t* s_free = bar_q + 1;                                         // [2]  128 arrivals: S(j) is in registers
  uint64_t* o_staged = s_free + 2;                                      //      128 arrivals: output rows are in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_staged + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(k_full + i, 1); mbar_init(v_full + i, 1); mbar_init(k_empty + i, 1); mbar_init(v_empty + i, 1);
    }
    mbar_init(bar_s, 1); mbar_init(bar_s + 1, 1);
    mbar_init(p_ready, 128); mbar_init(p_ready + 1, 128);
    mbar_init(bar_o, 1); mbar_init(bar_q, 1);
    mbar_init(s_free, 128); mbar_init(s_free + 1, 128); mbar_init(o_staged, 128);
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
  bool ok = true;
  CB_PHASE_DECL_T(128, 64);            // slot 0: the MMA / TMA thread, slot 1: a softmax thread

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer: Q once, then the K and V rings
    // (whole warp, warp-uniform control flow, one elected lane issues; see elect_one)
    const int u_start = __shfl_sync(0xffffffffu, start, 0);
    const int u_qb = __shfl_sync(0xffffffffu, qb, 0);
    const int u_nkv = __shfl_sync(0xffffffffu, n_kv, 0);
    if (elect_one()) {
      mbar_expect_tx(bar_q, L::QT);
#pragma unroll
      for (int p = 0; p < PANELS; ++p) tma_load_2d(sQ + p * 16384, &tmQ, bar_q, h * D + p * 64, u_start + u_qb * 128);
    }
    for (int j = 0; j < u_nkv && ok; ++j) {
      const int st = j % NS;
      if (j >= NS) {                                    // the stage's previous block: S(j - NS) complete
        ok = __all_sync(0xffffffffu, mbar_wait(k_empty + st, ((j / NS) - 1) & 1, abort_flag, a.status, CB_ERR_WAIT_EMPTY) && ok);
        if (!ok) break;
      }
      if (elect_one()) {
        mbar_expect_tx(k_full + st, L::KT);
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          tma_load_2d(sK + st * L::KT + p * 8192, &tmK, k_full + st, hkv * D + p * 64, u_start + j * 64);
      }
      if (j >= NS) {                                    // P V of block j - NS complete
        ok = __all_sync(0xffffffffu, mbar_wait(v_empty + st, ((j / NS) - 1) & 1, abort_flag, a.status, CB_ERR_WAIT_EMPTY) && ok);
        if (!ok) break;
      }
      if (elect_one()) {
        mbar_expect_tx(v_full + st, L::KT);
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          tma_load_2d(sV + st * L::KT + p * 8192, &tmV, v_full + st, hkv * D + p * 64, u_start + j * 64);
      }
    }
    __syncwarp();
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issue
    // Per kv block: wait for P(j), issue O += P(j) V(j), then S(j+2) into the score buffer P(j) has just left.
    // Every tcgen05.commit arrives on the consumers' barrier and on the ring's "stage free" barrier.
    const int u_nkv = __shfl_sync(0xffffffffu, n_kv, 0);
    const uint32_t u_tmem = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t qa = smem_u32(sQ);
    auto wait_w = [&](uint64_t* bar, uint32_t parity, int code) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, a.status, code) && ok);
    };
    auto issue_s = [&](int j) {                         // S(j) = Q K(j)^T into buffer j & 1
      const int st = j % NS;
      wait_w(k_full + st, (j / NS) & 1, CB_ERR_WAIT_FULL);
      const uint32_t kb = smem_u32(sK + st * L::KT);
      tc_fence_after();
      if (ok && elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16_ss(u_tmem + (j & 1) * 64, umma_smem_desc(qa + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                      umma_smem_desc(kb + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), IDESC_S, kk != 0);
        umma_commit(bar_s + (j & 1));
        umma_commit(k_empty + st);
      }
    };
    wait_w(bar_q, 0, CB_ERR_WAIT_FULL);
    if (ok) issue_s(0);
    if (ok && u_nkv > 1) issue_s(1);
    CB_PHASE(0);
    for (int j = 0; j < u_nkv && ok; ++j) {
      const int st = j % NS;
      if (P_APART && j + 2 < u_nkv) {
        wait_w(s_free + (j & 1), (j >> 1) & 1, CB_ERR_WAIT_TMEM_EMPTY);
        if (ok) issue_s(j + 2);
      }
      CB_PHASE(3);
      wait_w(p_ready + (j & 1), (j >> 1) & 1, CB_ERR_WAIT_TMEM_EMPTY);
      CB_PHASE(1);
      wait_w(v_full + st, (j / NS) & 1, CB_ERR_WAIT_FULL);
      CB_PHASE(2);
      if (!ok) break;
      tc_fence_after();
      const uint32_t vb = smem_u32(sV + st * L::KT);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)                  // O += P(j) V(j): A = P from TMEM, 16 bf16 = 8 words per step
          umma_f16_ts(u_tmem + C_O, u_tmem + (P_APART ? C_P + (j & 1) * 32 : (j & 1) * 64) + kk * 8,
                      umma_smem_desc(vb + kk * 2048, 8192, 1024), IDESC_PV, (j | kk) != 0);
        umma_commit(bar_o);
        umma_commit(v_empty + st);
      }
      CB_PHASE(4);
      if (!P_APART && j + 2 < u_nkv) issue_s(j + 2);
      CB_PHASE(8);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax: thread r owns score row r
    const int r = tid;
    const uint32_t t_row = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const float sl2 = a.scale * LOG2E;
    const float raise = FWD3_RAISE_LOG2 / sl2;          // in raw score units
    float m_ref = -INFINITY, l_run = 0.f;
    // every wait ends in a warp-wide vote, so that the lanes of a warp leave the loop together (the TMEM loads
    // and stores and the votes below want the whole warp)
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, a.status, code) && ok);
    };
    CB_PHASE(0);
    for (int j = 0; j < n_kv; ++j) {
      const uint32_t t_s = t_row + (j & 1) * 64;
      wait_all(bar_s + (j & 1), (j >> 1) & 1, CB_ERR_WAIT_TMEM_FULL);
      CB_PHASE(1);
      if (!ok) break;
      tc_fence_after();
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(t_s, s0);
      tmem_ld_32x32(t_s + 32, s1);
      tmem_ld_wait();
      if (P_APART) {                                    // the scores are in registers: their buffer may take S(j+2)
        tc_fence_before();
        mbar_arrive(s_free + (j & 1));
      }
      CB_PHASE(2);
      // columns j*64 + c <= qb*128 + r are visible; only the blocks that touch the diagonal need the test
      const int lim = qb * 128 + r - j * 64;
      if (j >= 2 * qb) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (c > lim) s0[c] = 0xff800000u;             // -inf
          if (c + 32 > lim) s1[c] = 0xff800000u;
        }
      }
      float mxc[8];                                     // eight independent chains: the maximum is latency-, not issue-bound
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        mxc[q] = fmaxf(__uint_as_float(s0[q]), __uint_as_float(s0[q + 4]));
        mxc[q + 4] = fmaxf(__uint_as_float(s1[q]), __uint_as_float(s1[q + 4]));
      }
#pragma unroll
      for (int c = 8; c < 32; c += 4) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          mxc[q] = fmaxf(mxc[q], __uint_as_float(s0[c + q]));
          mxc[q + 4] = fmaxf(mxc[q + 4], __uint_as_float(s1[c + q]));
        }
      }
      const float mx = fmaxf(fmaxf(fmaxf(mxc[0], mxc[1]), fmaxf(mxc[2], mxc[3])), fmaxf(fmaxf(mxc[4], mxc[5]), fmaxf(mxc[6], mxc[7])));
      CB_PHASE(3);
      const bool up = mx > m_ref + raise;               // also true for the first block (m_ref = -inf)
      bool o_seen = false;
      if (__any_sync(0xffffffffu, up)) {
        if (j > 0) {
          // my O row is rescaled in TMEM: P V of block j - 1 has to be complete, and that of block j cannot start
          // before this thread has signalled p_ready
          wait_all(bar_o, (j - 1) & 1, CB_ERR_WAIT_TMEM_FULL);
          o_seen = true;
          if (!ok) break;
          tc_fence_after();
          const float alpha = up ? ex2_approx((m_ref - mx) * sl2) : 1.f;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_row + C_O + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_row + C_O + c * 32, o);
          }
          l_run *= alpha;
        }
        if (up) m_ref = mx;
      }
      CB_PHASE(4);
      const float mb = m_ref * sl2;
      uint32_t pk[32];
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float e0 = ex2_approx(fmaf(__uint_as_float(s0[2 * i]), sl2, -mb));
        // three exponentials in eight run on the FMA pipe: the exp2 unit is this loop's bound
        const float x1 = fmaf(__uint_as_float(s0[2 * i + 1]), sl2, -mb);
        const float e1 = (i & 1) ? ex2_fma(x1) : ex2_approx(x1);
        const float e2 = ex2_approx(fmaf(__uint_as_float(s1[2 * i]), sl2, -mb));
        const float e3 = ex2_fma(fmaf(__uint_as_float(s1[2 * i + 1]), sl2, -mb));
        rs0 += e0 + e1;
        rs1 += e2 + e3;
        pk[i] = pack_bf16x2(e0, e1);
        pk[16 + i] = pack_bf16x2(e2, e3);
      }
      l_run += rs0 + rs1;
      CB_PHASE(5);
      // P(j): 64 bf16 = 32 words, over the scores just read or (D = 64) in its own columns, which P V of block
      // j - 2 has left: its completion was observed before the arrival of the last iteration
      tmem_st_32x32(P_APART ? t_row + C_P + (j & 1) * 32 : t_s, pk);
      tmem_st_wait();
      CB_PHASE(6);
      if (j > 0 && !o_seen) {
        // keep pace with bar_o: a parity wait can only tell the current phase from the one before it (a lane
        // that gives up here is caught by the vote of the next wait)
        ok &= mbar_wait(bar_o, (j - 1) & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
      }
      CB_PHASE(7);
      tc_fence_before();
      mbar_arrive(p_ready + (j & 1));
      CB_PHASE(8);
    }
    // A block that lies wholly inside its document leaves through shared memory and a TMA store (below)
    const bool whole = a.o_tma != 0 && (qb + 1) * 128 <= len;          // CTA-uniform
    if (ok) {
      wait_all(bar_o, (n_kv - 1) & 1, CB_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      const int rg = qb * 128 + r;
      const bool row_ok = rg < len;                     // the TMEM loads below are warp-wide; only the stores are per row
      const float inv = 1.f / l_run;
      const long long t = start + (row_ok ? rg : 0);
      CB_DEBUG_CHECK_ST(a.status, t >= 0 && t < a.T, CB_DBG_ATTN_ROW, t);
      // A block that lies wholly inside its document leaves through shared memory (the Q tile, which the last
      // S product has finished with) and one TMA store per 64-column panel: row-contiguous 128-byte writes
      // instead of 32 scattered 16-byte sectors per store instruction.  The last, partial block of a document
      // stores row by row, because a TMA box cannot skip the rows that belong to the next document.
      uint4* op = reinterpret_cast<uint4*>(a.O + t * a.ldo + static_cast<long long>(h) * D);
      if (ok) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(t_row + C_O + c * 32, o);
          tmem_ld_wait();
          if (whole) {
            float v[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = __uint_as_float(o[q]) * inv;
            store_row_chunk32(sQ, r, c, v);
          } else if (row_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(o[8 * q + 0]) * inv, __uint_as_float(o[8 * q + 1]) * inv);
              u.y = pack_bf16x2(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv);
              u.z = pack_bf16x2(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv);
              u.w = pack_bf16x2(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv);
              op[c * 4 + q] = u;
            }
          }
        }
        if (row_ok) a.lse[static_cast<long long>(h) * a.T + t] = m_ref * a.scale + __logf(l_run);
      }
    }
    if (whole) {
      // every softmax thread reports its rows staged (also one that gave up, so that nobody waits without a
      // limit); warp 0 then stores the tile
      fence_async_smem();
      mbar_arrive(o_staged);
      if (warp == 0) {
        wait_all(o_staged, 0, CB_ERR_WAIT_MISC);
        if (ok && elect_one()) {
#pragma unroll
          for (int p = 0; p < PANELS; ++p) tma_store_2d(&tmO, sQ + p * 16384, h * D + p * 64, start + qb * 128);
          tma_store_commit();
          tma_store_wait_all();                         // shared memory is released when the CTA exits
        }
      }
    }
  }
  CB_PHASE(9);
  CB_PHASE_FLUSH;
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
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
  static constexpr int NQ = (D == 128) ? 2 : 1;       // Q / dO stages: D = 128 runs one CTA per SM and has the room to
                                                      // fetch the next query block while this one is worked on
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;              // NQ stages
  static constexpr int OFF_DO = (2 + NQ) * TILE;      // NQ stages
  static constexpr int OFF_P = (2 + 2 * NQ) * TILE;   // P, then dS (bf16 [128 x 128] operand image)
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
  if (!locate_tile(a.cu, a.n_docs, blockIdx.y, start, len, jb, nblk)) return;
  jb = nblk - jb;                                      // weight = query blocks from the diagonal on = nblk - jb
  const int h = blockIdx.x;
  const int hkv = h / (a.hq / a.hk);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sdO = smem + L::OFF_DO;
  uint8_t* sP = smem + L::OFF_P;
  constexpr int NQ = L::NQ;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);   // [2]
  uint64_t* bar_kv = q_full + 2;
  uint64_t* bar_s = q_full + 3;
  uint64_t* bar_dp = q_full + 4;
  uint64_t* bar_dq = q_full + 5;
  uint64_t* stg_free = q_full + 6;                   // the dQ tile of the last iteration has left shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // 8 warps: warps w and w + 4 own the same 32 TMEM lanes (score rows) and split the columns in halves,
  // which doubles the number of warps available to hide TMEM / shared-memory latency
  const int tid = threadIdx.x, warp = tid >> 5;
  const int q4 = warp & 3, half = warp >> 2;
  if (tid == 0) {
    mbar_init(q_full, 1); mbar_init(q_full + 1, 1); mbar_init(bar_kv, 1); mbar_init(bar_s, 1); mbar_init(bar_dp, 1); mbar_init(bar_dq, 1);
    mbar_init(stg_free, 1);
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

  const int n_it = nblk - jb;
  // Warp 0 issues every TMA load and MMA: the whole warp follows the issuing path with warp-uniform control flow
  // and one elected lane issues, with the values that feed coordinates and descriptors broadcast from lane 0, so
  // that the compiler can keep them in uniform registers.
  const bool w0 = __shfl_sync(0xffffffffu, warp, 0) == 0;
  const int u_start = __shfl_sync(0xffffffffu, start, 0);
  const int u_jb = __shfl_sync(0xffffffffu, jb, 0);
  const int kv_row0 = u_start + u_jb * 128;
  auto load_q = [&](int it) {                          // Q / dO of query block jb + it into stage it % NQ
    const int row0 = u_start + (u_jb + it) * 128;
    const int st = it % NQ;
    mbar_expect_tx(q_full + st, 2 * L::TILE);
#pragma unroll
    for (int p = 0; p < PANELS; ++p) {
      tma_load_2d(sQ + st * L::TILE + p * 16384, &tmQ, q_full + st, h * D + p * 64, row0);
      tma_load_2d(sdO + st * L::TILE + p * 16384, &tmdO, q_full + st, h * D + p * 64, row0);
    }
  };

  bool ok = true;
  if (w0) {
    if (elect_one()) {
      mbar_expect_tx(bar_kv, 2 * L::TILE);
#pragma unroll
      for (int p = 0; p < PANELS; ++p) {
        tma_load_2d(sK + p * 16384, &tmK, bar_kv, hkv * D + p * 64, kv_row0);
        tma_load_2d(sV + p * 16384, &tmV, bar_kv, hkv * D + p * 64, kv_row0);
      }
      load_q(0);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar_kv, 0, abort_flag, a.status, CB_ERR_WAIT_FULL));
  }

  const int r = q4 * 32 + (tid & 31);
  const float sl2 = a.scale * LOG2E;
  const uint32_t kA = smem_u32(sK), vA = smem_u32(sV), pA = smem_u32(sP);
  const uint32_t u_tmem = __shfl_sync(0xffffffffu, tmem, 0);
  // lse and delta of my query row: fetched one iteration ahead, the loads fly while this iteration works
  // (the loaded values are not touched before the next iteration, so nothing waits for the loads here)
  auto row_stats = [&](int it, float& lse_o, float& dlt_o) {
    const int rg_ = (jb + it) * 128 + r;
    const long long at = static_cast<long long>(h) * a.T + start + rg_;
    lse_o = 0.f;
    dlt_o = 0.f;
    if (it < n_it && rg_ < len) {
      lse_o = __ldg(a.lse + at);
      dlt_o = __ldg(a.delta + at);
    }
  };
  float lse_n, dlt_n;
  row_stats(0, lse_n, dlt_n);

  CB_PHASE_DECL;
  for (int it = 0; it < n_it; ++it) {
    const int i = jb + it;
    CB_PHASE(0);
    const uint32_t qA = smem_u32(sQ + (it % NQ) * L::TILE), doA = smem_u32(sdO + (it % NQ) * L::TILE);
    if (w0) {
      ok = __all_sync(0xffffffffu, mbar_wait(q_full + (it % NQ), (it / NQ) & 1, abort_flag, a.status, CB_ERR_WAIT_FULL) && ok);
      tc_fence_after();
      if (elect_one()) {
        if (ok) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            umma_f16_ss(u_tmem + C_S, desc_kmajor(qA, kk), desc_kmajor(kA, kk), IDESC_S, kk != 0);
          umma_commit(bar_s);
        }
        // While S is computed, the TMA reduce of the last iteration's dQ tile finishes reading the P / dS buffer
        // (and, D = 128, the dO stage the next load goes to); everybody waits for `stg_free` before writing P.
        tma_store_wait_read<0>();
        if (NQ == 2 && ok && it + 1 < n_it) load_q(it + 1);
        mbar_arrive(stg_free);
      }
    }
    const int rg = i * 128 + r;                      // my query row within the document
    const bool row_ok = rg < len;
    const float lse2 = row_ok ? lse_n * LOG2E : INFINITY, dlt = dlt_n;
    row_stats(it + 1, lse_n, dlt_n);
    const bool diag = (it == 0);
    CB_PHASE(1);
    // ---- phase 1: P = exp(S - lse), masked, to shared memory
    ok &= mbar_wait(bar_s, it & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    ok &= mbar_wait(stg_free, it & 1, abort_flag, a.status, CB_ERR_WAIT_MISC);
    tc_fence_after();
    CB_PHASE(2);
    // my 64 probabilities stay in registers as bf16 pairs (pk) for phase 2; rows past the end of the document
    // carry lse = +inf and so exponentiate to exact zeros, only the diagonal block tests columns against rows
    uint32_t pk[2][16];
#pragma unroll
    for (int cl = 0; cl < 2; ++cl) {
      const int c = half * 2 + cl;
      uint32_t s[32];
      tmem_ld_32x32(t_row + C_S + c * 32, s);
      tmem_ld_wait();
      if (diag) {
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          float e0 = ex2_approx(fmaf(__uint_as_float(s[2 * k]), sl2, -lse2));
          float e1 = ex2_approx(fmaf(__uint_as_float(s[2 * k + 1]), sl2, -lse2));
          e0 = (c * 32 + 2 * k <= r) ? e0 : 0.f;
          e1 = (c * 32 + 2 * k + 1 <= r) ? e1 : 0.f;
          pk[cl][k] = pack_bf16x2(e0, e1);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 16; ++k) {                  // one exponential in four on the FMA pipe (see ex2_fma)
          const float x1 = fmaf(__uint_as_float(s[2 * k + 1]), sl2, -lse2);
          pk[cl][k] = pack_bf16x2(ex2_approx(fmaf(__uint_as_float(s[2 * k]), sl2, -lse2)),
                                  (k & 1) ? ex2_fma(x1) : ex2_approx(x1));
        }
      }
      store_row_chunk32_packed(sP, r, c, pk[cl]);
    }
    CB_PHASE(3);
    tc_fence_before();
    fence_async_smem();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    CB_PHASE(4);
    if (w0) {
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)                // dV += P^T dO     (K = the 128 query rows)
          umma_f16_ss(u_tmem + C_DV, desc_mnmajor(pA, kk), desc_mnmajor(doA, kk), IDESC_T, (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)           // dP = dO V^T      (over the columns S occupied)
          umma_f16_ss(u_tmem + C_S, desc_kmajor(doA, kk), desc_kmajor(vA, kk), IDESC_S, kk != 0);
        umma_commit(bar_dp);
      }
    }
    // ---- phase 2: dS = P (dP - delta) scale, overwriting P in shared memory
    CB_PHASE(5);
    ok &= mbar_wait(bar_dp, it & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    CB_PHASE(6);
#pragma unroll
    for (int cl = 0; cl < 2; ++cl) {
      const int c = half * 2 + cl;
      uint32_t dp[32];
      tmem_ld_32x32(t_row + C_S + c * 32, dp);
      tmem_ld_wait();
      uint32_t ds[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float2 pp = unpack_bf16x2(pk[cl][k]);
        ds[k] = pack_bf16x2(pp.x * (__uint_as_float(dp[2 * k]) - dlt) * a.scale,
                            pp.y * (__uint_as_float(dp[2 * k + 1]) - dlt) * a.scale);
      }
      store_row_chunk32_packed(sP, r, c, ds);
    }
    CB_PHASE(7);
    tc_fence_before();
    fence_async_smem();
    if (__syncthreads_or(!ok)) { ok = false; break; }
    CB_PHASE(8);
    if (w0) {
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)                // dK += dS^T Q
          umma_f16_ss(u_tmem + C_DK, desc_mnmajor(pA, kk), desc_mnmajor(qA, kk), IDESC_T, (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)                // dQ = dS K        (K = the 128 kv rows)
          umma_f16_ss(u_tmem + C_S, desc_kmajor(pA, kk), desc_mnmajor(kA, kk), IDESC_DQ, kk != 0);
        umma_commit(bar_dq);
      }
    }
    // ---- phase 3: dQ out
    CB_PHASE(9);
    ok &= mbar_wait(bar_dq, it & 1, abort_flag, a.status, CB_ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    CB_PHASE(10);
    if (NQ == 1 && w0 && ok && it + 1 < n_it) {                         // Q / dO of this iteration are consumed
      if (elect_one()) load_q(it + 1);
    }
    {
      // dQ tile (fp32) -> shared memory as [128 x 32] boxes in the layout of the dq_acc tensor map -> one TMA
      // reduce-add per box instead of eight red.global.add per thread and box.  The first two boxes go to the
      // P / dS buffer, which nobody reads any more; D = 128 has two more, which go to this iteration's dO stage
      // (dV and dP have consumed it; the next load into that stage waits for the reduce's reads, see the loop top).
      // Rows past the end of the document carry exact zeros (their P was masked), rows past T are clipped.
      uint8_t* sdO_it = sdO + (it % NQ) * L::TILE;
#pragma unroll
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t dq[32];
        tmem_ld_32x32(t_row + C_S + c * 32, dq);
        tmem_ld_wait();
        uint8_t* dstrow = (c < 2 ? sP + c * 16384 : sdO_it + (c - 2) * 16384) + r * 128;
#pragma unroll
        for (int cc = 0; cc < 8; ++cc)
          *reinterpret_cast<uint4*>(dstrow + ((cc ^ (r & 7)) << 4)) = make_uint4(dq[4 * cc], dq[4 * cc + 1], dq[4 * cc + 2], dq[4 * cc + 3]);
      }
      CB_PHASE(11);
      fence_async_smem();
      tc_fence_before();
      if (__syncthreads_or(!ok)) { ok = false; break; }
      CB_PHASE(12);
      if (w0 && elect_one()) {
        CB_DEBUG_CHECK_ST(a.status, start + i * 128 >= 0 && ((h * D) * 4) % 16 == 0, CB_DBG_TMA_COORD, start + i * 128);
#pragma unroll
        for (int c = 0; c < D / 32; ++c)
          tma_reduce_add_2d(&tmdQ, c < 2 ? sP + c * 16384 : sdO_it + (c - 2) * 16384, h * D + c * 32,
                            u_start + (u_jb + it) * 128);
        tma_store_commit();
      }
    }
  }
  CB_PHASE_FLUSH;
  if (w0) {
    if (elect_one()) tma_store_wait_all();
  }
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
__global__ void attn_bwd_finalize_kernel(float* __restrict__ dq_acc, float* __restrict__ dk_part,
                                         float* __restrict__ dv_part, bf16* __restrict__ dqkv, long long ld,
                                         int T, int hq, int hk, int D, const int* __restrict__ cu, int n_docs,
                                         int part_heads, int clear) {
  // part_heads: heads per token in dk_part / dv_part — hq (one partial per query head, summed here) or hk
  // (already accumulated per kv head by the kernel).  clear: write zeros back over every accumulator value read, so
  // that a caller who keeps the scratch buffers between calls never has to clear them again.
  const long long t = blockIdx.x;
  const int nq = hq * D, nk = hk * D, g = part_heads / hk;
  bf16* out = dqkv + t * ld;
  const bool valid = t < cu[n_docs];                  // padding tokens get zero gradients
  for (int c = threadIdx.x * 4; c < nq + 2 * nk; c += blockDim.x * 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
      if (c < nq) {
        v = *reinterpret_cast<const float4*>(dq_acc + t * nq + c);
        if (clear) *reinterpret_cast<float4*>(dq_acc + t * nq + c) = make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        const int cc = (c - nq) % nk, which = (c - nq) / nk;
        const int kvh = cc / D, d = cc % D;
        float* src = (which == 0 ? dk_part : dv_part) + (t * part_heads + static_cast<long long>(kvh) * g) * D + d;
        for (int i = 0; i < g; ++i) {
          const float4 x = *reinterpret_cast<const float4*>(src + static_cast<long long>(i) * D);
          v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
          if (clear) *reinterpret_cast<float4*>(src + static_cast<long long>(i) * D) = make_float4(0.f, 0.f, 0.f, 0.f);
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
// o [T, hq, D] with pitch ldo; lse [hq, T] fp32.  Rows of o at or beyond cu[n_docs] (padding) are written as
// zeros by the kernel, their lse entries are left untouched.  D is 64 or 128, hq a multiple of hk.
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
  dim3 grid(hq, (T + 127) / 128 + n_docs);            // x: query head (fastest, the heads of a group share K/V in L2); y: tile by descending weight
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Default: the pipelined kernel (64-row kv blocks, double-buffered scores, O accumulated in TMEM).
  // CB_ATTN_FWD=1 in the environment selects the first form (one thread per row, 128-row kv blocks, O in
  // registers), CB_ATTN_FWD=2 the two-threads-per-row form; both are kept for comparison.
  static const int form = [] { const char* v = getenv("CB_ATTN_FWD"); return (v != nullptr && v[0] >= '1' && v[0] <= '3') ? v[0] - '0' : 3; }();
  if (form == 3) {
    CUtensorMap mk64, mv64;                             // K / V in boxes of 64 rows
    e = cbhost::make_tmap(&mk64, k, static_cast<unsigned long long>(hk) * D, T, ldk, 64, 64);
    if (e) return e;
    e = cbhost::make_tmap(&mv64, v, static_cast<unsigned long long>(hk) * D, T, ldv, 64, 64);
    if (e) return e;
    CUtensorMap mo;                                     // O in boxes of 128 rows x 64 columns, for the tile stores
    a.o_tma = cbhost::make_tmap(&mo, o, static_cast<unsigned long long>(hq) * D, T, ldo, 64, 128) == 0 ? 1 : 0;
    if (!a.o_tma) mo = mq;                              // O is not TMA-addressable: every block stores row by row
    if (D == 64) {
      static bool cfg = false;
      if (!cfg) { e = set_smem(cb::attn_fwd3_kernel<64>, cb::Fwd3Smem<64>::TOTAL); if (e) return e; cfg = true; }
      cb::attn_fwd3_kernel<64><<<grid, cb::FWD3_THREADS, cb::Fwd3Smem<64>::TOTAL, s>>>(mq, mk64, mv64, mo, a);
    } else {
      static bool cfg = false;
      if (!cfg) { e = set_smem(cb::attn_fwd3_kernel<128>, cb::Fwd3Smem<128>::TOTAL); if (e) return e; cfg = true; }
      cb::attn_fwd3_kernel<128><<<grid, cb::FWD3_THREADS, cb::Fwd3Smem<128>::TOTAL, s>>>(mq, mk64, mv64, mo, a);
    }
    return static_cast<int>(cudaGetLastError());
  }
  const bool two_thread_rows = form == 2;
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
                float* dv_part, void* dqkv, long long ld_dqkv, int* status, void* stream, int scratch_is_zero) {
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
  // scratch_is_zero: the caller keeps dq_acc / dk_part / dv_part between calls; they arrive all zero and the finalize
  // kernel leaves them all zero again, so the three clears are skipped
  if (!scratch_is_zero) CB_CHECK_CUDA(cudaMemsetAsync(dq_acc, 0, sizeof(float) * static_cast<size_t>(T) * hq * D, s));
  cb::AttnArgs a = {};
  a.T = T; a.hq = hq; a.hk = hk; a.n_docs = n_docs; a.cu = cu; a.scale = scale;
  a.lse = const_cast<float*>(lse); a.delta = delta; a.dq_acc = dq_acc; a.dk_part = dk_part; a.dv_part = dv_part;
  a.status = status;
  dim3 grid(hq, (T + 127) / 128 + n_docs);            // x: query head (fastest, the heads of a group share K/V in L2); y: tile by descending weight
  // Two threads per score row, S / dP / dQ sharing TMEM columns, dK / dV accumulated per kv head with red.add
  // (so those buffers start from zero).  D = 64 additionally fits two CTAs per SM.
  const int part_heads = hk;
  if (!scratch_is_zero) {
    CB_CHECK_CUDA(cudaMemsetAsync(dk_part, 0, sizeof(float) * static_cast<size_t>(T) * hk * D, s));
    CB_CHECK_CUDA(cudaMemsetAsync(dv_part, 0, sizeof(float) * static_cast<size_t>(T) * hk * D, s));
  }
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
                                                  hq, hk, D, cu, n_docs, part_heads, scratch_is_zero ? 1 : 0);
  return static_cast<int>(cudaGetLastError());
}

#ifdef CB_ATTN_PHASE_TIMERS
// out[2][16] cycles per phase (see CB_PHASE in attn_bwd2_kernel), slot 15 = number of CTAs; clears the table
int cb_attn_phase_read(unsigned long long* out) {
  CB_CHECK_CUDA(cudaDeviceSynchronize());
  CB_CHECK_CUDA(cudaMemcpyFromSymbol(out, cb::cb_attn_phase, sizeof(unsigned long long) * 32));
  unsigned long long zero[32] = {};
  CB_CHECK_CUDA(cudaMemcpyToSymbol(cb::cb_attn_phase, zero, sizeof(zero)));
  return 0;
}
#endif

}  // extern "C"
