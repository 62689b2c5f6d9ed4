// Collectives fused with their neighbouring compute, written as plain loads and stores on peer
// memory (NVLink 5 through NVSwitch gives every GPU a direct path to every peer's HBM).  No NCCL
// call is involved on these paths; the host only hands each kernel a table of peer pointers.
//
//   symm_barrier_kernel      all-rank barrier with a small fp32 payload per rank (epoch flags in
//                            each rank's flag pad, st.release.sys / ld.acquire.sys, bounded spin)
//   rs_reduce_sqnorm_kernel  data-parallel gradient reduce-scatter: every rank pulls its 1/W slice
//                            of the bucket from all W ranks, sums in fp32, scales by 1/W, keeps the
//                            fp32 result locally and produces sum-of-squares partials for clipping
//   adamw_shard_allgather_kernel
//                            AdamW on the owned slice (moments exist only for that slice) and the
//                            all-gather fused into the update: the new bf16 parameters are stored
//                            straight into every rank's parameter buffer
//
// Waits never spin unbounded: after the limit the kernel records an error in the status word and
// returns; the host raises on the next status check.  The reference is single-GPU and has no
// counterpart for any of this.
#include <cstring>
#include "common.cuh"

namespace cb {

constexpr int COMM_THREADS = 256;
constexpr int MAX_RANKS = 16;

struct PeerTable {
  void* ptr[MAX_RANKS];
};

// Flag pad layout per rank: [0, W) u64 epoch flags written by rank r into slot r;
// [MAX_RANKS, MAX_RANKS + W * PAYLOAD) fp32 payload slots (as u64 words: 2 floats each).
constexpr int PAYLOAD_FLOATS = 4;

// One block.  Thread r (< W): publish my payload and epoch into rank r's pad, then wait until rank r's
// epoch shows up in my pad.  `payload_in` (device, PAYLOAD_FLOATS floats) may be null.
// `gathered_out` (device, W * PAYLOAD_FLOATS floats) receives every rank's payload; may be null.
//
// The epoch is a device-resident counter advanced by the kernel itself (every rank runs the same
// sequence of barriers, so the counters agree); nothing about it is baked into the launch, which
// keeps the barrier correct when the launch is replayed from a CUDA graph.
__global__ void symm_barrier_kernel(PeerTable pads, int my_rank, int W, unsigned long long* __restrict__ epoch_ctr,
                                    const float* __restrict__ payload_in, float* __restrict__ gathered_out,
                                    unsigned long long wait_limit_ns, int* status) {
  // no shared memory in this kernel or in rs_bucket_kernel: they run beside persistent GEMM CTAs that leave an SM
  // little more than the per-CTA reserve, and an SM that cannot take one of those CTAs delays the whole GEMM
  const unsigned long long epoch = *epoch_ctr + 1;       // every thread reads the counter before thread 0 advances it
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = epoch;
  if (status[0] != 0) return;
  const int r = threadIdx.x;
  if (r < W) {
    unsigned long long* peer_pad = static_cast<unsigned long long*>(pads.ptr[r]);
    float* peer_payload = reinterpret_cast<float*>(peer_pad + MAX_RANKS) + my_rank * PAYLOAD_FLOATS;
    if (payload_in != nullptr) {
#pragma unroll
      for (int i = 0; i < PAYLOAD_FLOATS; ++i) peer_payload[i] = payload_in[i];
    }
    __threadfence_system();
    st_release_sys_u64(peer_pad + my_rank, epoch);
    // wait for rank r's arrival in my own pad
    const unsigned long long* mine = static_cast<const unsigned long long*>(pads.ptr[my_rank]) + r;
    const uint64_t t0 = globaltimer_ns();
    bool ok = true;
    while (ld_acquire_sys_u64(mine) < epoch) {
      if (globaltimer_ns() - t0 > wait_limit_ns) {
        atomicCAS(status, 0, CB_ERR_WAIT_PEER);
        status[1] = r;
        status[2] = my_rank;
        ok = false;
        break;
      }
      __nanosleep(64);
    }
    if (ok && gathered_out != nullptr) {
      const float* src = reinterpret_cast<const float*>(
                             static_cast<const unsigned long long*>(pads.ptr[my_rank]) + MAX_RANKS) + r * PAYLOAD_FLOATS;
#pragma unroll
      for (int i = 0; i < PAYLOAD_FLOATS; ++i) gathered_out[r * PAYLOAD_FLOATS + i] = src[i];
    }
  }
}

__device__ __forceinline__ void acc_bf16x8(const uint4& u, float (&a)[8]) {
  const float2 x0 = unpack_bf16x2(u.x), x1 = unpack_bf16x2(u.y), x2 = unpack_bf16x2(u.z), x3 = unpack_bf16x2(u.w);
  a[0] += x0.x; a[1] += x0.y; a[2] += x1.x; a[3] += x1.y; a[4] += x2.x; a[5] += x2.y; a[6] += x3.x; a[7] += x3.y;
}

// reduced[i - lo] = (1/W) * sum_r grads[r][i]  for i in [lo, hi)  (bf16 in, fp32 out);
// partials[block] = sum of squares of this block's reduced values.  lo and hi are multiples of 8.
__global__ void __launch_bounds__(COMM_THREADS)
rs_reduce_sqnorm_kernel(PeerTable grads, int W, long long lo, long long hi, float* __restrict__ reduced,
                        float* __restrict__ partials, int* status) {
  __shared__ float sred[COMM_THREADS / 32];
  float sq = 0.f;
  CB_DEBUG_CHECK_ST(status, ((lo | hi) & 7) == 0 && hi >= lo, CB_DBG_COMM_SLICE, lo);
  if (status[0] == 0) {
    const float inv = 1.f / static_cast<float>(W);
    const long long nvec = (hi - lo) >> 3;
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < W; ++r) {
        const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const bf16*>(grads.ptr[r]) + lo + (v << 3));
        acc_bf16x8(u, a);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] *= inv;
        sq += a[j] * a[j];
      }
      float4* o = reinterpret_cast<float4*>(reduced + (v << 3));
      o[0] = make_float4(a[0], a[1], a[2], a[3]);
      o[1] = make_float4(a[4], a[5], a[6], a[7]);
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < COMM_THREADS / 32 ? sred[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
}

// payload[0] = sum(partials[0..n))   (single block, deterministic order)
__global__ void sum_partials_kernel(const float* __restrict__ partials, int n, float* __restrict__ payload) {
  __shared__ double sred[32];
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += static_cast<double>(partials[i]);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += sred[i];
    payload[0] = static_cast<float>(t);
    payload[1] = payload[2] = payload[3] = 0.f;
  }
}

// Per-bucket reduce-scatter that runs beside the backward pass on a second stream.  Same arithmetic as
// rs_reduce_sqnorm_kernel, shaped to share SMs with the compute kernels: 128 threads per block and a
// grid chosen by the host, one 16-byte vector per thread and pass with all ranks' loads in flight.  partials[block]
// receives each warp's sum of squares (RSB_THREADS / 32 slots per block); the host sums all buckets' partials once
// after the last bucket.
constexpr int RSB_THREADS = 128;
__global__ void __launch_bounds__(RSB_THREADS)
rs_bucket_kernel(PeerTable grads, int W, long long lo, long long hi, float* __restrict__ reduced,
                 float* __restrict__ partials, int* status) {
  float sq = 0.f;
  CB_DEBUG_CHECK_ST(status, ((lo | hi) & 7) == 0 && hi >= lo, CB_DBG_COMM_SLICE, lo);
  if (status[0] == 0) {
    const float inv = 1.f / static_cast<float>(W);
    const long long nvec = (hi - lo) >> 3;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    // One 16-byte vector per thread and pass, with the loads from up to eight ranks in flight at once (at eight
    // ranks two loads per pass left the links at a third of their rate); the sum runs over the ranks in rank
    // order, so every rank computes bit-identical values for its slice whatever the grid.
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec; v += stride) {
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r0 = 0; r0 < W; r0 += 8) {
        uint4 u[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (r0 + k < W) u[k] = *reinterpret_cast<const uint4*>(static_cast<const bf16*>(grads.ptr[r0 + k]) + lo + (v << 3));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (r0 + k < W) acc_bf16x8(u[k], a);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] *= inv;
        sq += a[j] * a[j];
      }
      float4* o = reinterpret_cast<float4*>(reduced + (v << 3));
      o[0] = make_float4(a[0], a[1], a[2], a[3]);
      o[1] = make_float4(a[4], a[5], a[6], a[7]);
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) partials[blockIdx.x * (RSB_THREADS / 32) + (threadIdx.x >> 5)] = sq;   // one slot per warp
}

// AdamW on the owned slice [lo, hi) and fused all-gather.  `gathered` holds every rank's payload
// (slot 0 = its share of the squared gradient norm); the clip coefficient is computed from their sum
// in rank order, so all ranks get the same value.  chunk_group[(i - lo) / 1024] selects the
// hyper-parameter row (lr, wd, beta1, beta2, eps, bc1, bc2, -) of element i.
__global__ void __launch_bounds__(COMM_THREADS)
adamw_shard_allgather_kernel(PeerTable params, int W, int my_rank, long long lo, long long hi,
                             const float* __restrict__ reduced, float* __restrict__ m, float* __restrict__ v,
                             float* __restrict__ master, const unsigned char* __restrict__ chunk_group,
                             const float* __restrict__ hyper, const float* __restrict__ gathered, float max_norm,
                             float* __restrict__ norm_out, int W_store, const long long* __restrict__ chunk_off,
                             int* status) {
  if (status[0] != 0) return;
  float tot = 0.f;
  for (int r = 0; r < W; ++r) tot += gathered[r * PAYLOAD_FLOATS];
  const float norm = sqrtf(tot);
  const float clip = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0 && norm_out != nullptr) {
    norm_out[0] = tot;
    norm_out[1] = norm;
    norm_out[2] = clip;
  }
  const long long nvec = (hi - lo) >> 3;
  const bf16* mine = static_cast<const bf16*>(params.ptr[my_rank]);
  for (long long vi = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; vi < nvec;
       vi += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = vi << 3;
    // bucketed layout: the owned slice is a concatenation of one piece per bucket; chunk_off[c] is where the
    // c-th 1024-element chunk of the slice sits in the flat parameter buffer.  Without the table: lo + e.
    const long long ge = chunk_off != nullptr ? chunk_off[e >> 10] + (e & 1023) : lo + e;
    const float* h = hyper + chunk_group[e >> 10] * 8;
    const float lr = h[0], wd = h[1], b1 = h[2], b2 = h[3], eps = h[4], bc1 = h[5], bc2 = h[6];
    const float step = lr / bc1, inv_bc2 = 1.f / bc2, decay = 1.f - lr * wd;
    float g[8], w[8], mm[8], vv[8];
    const float4 g0 = *reinterpret_cast<const float4*>(reduced + e), g1 = *reinterpret_cast<const float4*>(reduced + e + 4);
    g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
    if (master != nullptr) {
      const float4 w0 = *reinterpret_cast<const float4*>(master + e), w1 = *reinterpret_cast<const float4*>(master + e + 4);
      w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
    } else {
      const uint4 u = *reinterpret_cast<const uint4*>(mine + ge);
      const float2 x0 = unpack_bf16x2(u.x), x1 = unpack_bf16x2(u.y), x2 = unpack_bf16x2(u.z), x3 = unpack_bf16x2(u.w);
      w[0] = x0.x; w[1] = x0.y; w[2] = x1.x; w[3] = x1.y; w[4] = x2.x; w[5] = x2.y; w[6] = x3.x; w[7] = x3.y;
    }
    const float4 m0 = *reinterpret_cast<const float4*>(m + e), m1 = *reinterpret_cast<const float4*>(m + e + 4);
    const float4 v0 = *reinterpret_cast<const float4*>(v + e), v1 = *reinterpret_cast<const float4*>(v + e + 4);
    mm[0] = m0.x; mm[1] = m0.y; mm[2] = m0.z; mm[3] = m0.w; mm[4] = m1.x; mm[5] = m1.y; mm[6] = m1.z; mm[7] = m1.w;
    vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * clip;
      float x = w[j] * decay;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      x -= step * mm[j] / (sqrtf(vv[j] * inv_bc2) + eps);
      w[j] = x;
    }
    *reinterpret_cast<float4*>(m + e) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(m + e + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    *reinterpret_cast<float4*>(v + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(v + e + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    if (master != nullptr) {
      *reinterpret_cast<float4*>(master + e) = make_float4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<float4*>(master + e + 4) = make_float4(w[4], w[5], w[6], w[7]);
    }
    uint4 o;
    o.x = pack_bf16x2(w[0], w[1]); o.y = pack_bf16x2(w[2], w[3]);
    o.z = pack_bf16x2(w[4], w[5]); o.w = pack_bf16x2(w[6], w[7]);
    for (int r = 0; r < W_store; ++r)      // the all-gather: every rank receives the updated slice
      *reinterpret_cast<uint4*>(static_cast<bf16*>(params.ptr[(my_rank + r) % W]) + ge) = o;
  }
}

// out[i] = sum_r bufs[r][i] * scale over [0, n) (bf16), every rank computes the full result from
// peer loads (small tensors: LoRA gradients, scalars).  n a multiple of 8.
__global__ void __launch_bounds__(COMM_THREADS)
allreduce_pull_kernel(PeerTable bufs, int W, long long n, float scale, bf16* __restrict__ out, int* status) {
  if (status[0] != 0) return;
  const long long nvec = n >> 3;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < W; ++r)
      acc_bf16x8(*reinterpret_cast<const uint4*>(static_cast<const bf16*>(bufs.ptr[r]) + (v << 3)), a);
    uint4 o;
    o.x = pack_bf16x2(a[0] * scale, a[1] * scale); o.y = pack_bf16x2(a[2] * scale, a[3] * scale);
    o.z = pack_bf16x2(a[4] * scale, a[5] * scale); o.w = pack_bf16x2(a[6] * scale, a[7] * scale);
    *reinterpret_cast<uint4*>(out + (v << 3)) = o;
  }
}


// ------------------------------------------------------------------------------------------------------
// Tensor/sequence parallel: all-gather by push, fused with the producing RMSNorm.
//
// y[row] = x[row] * rstd(row) * (offset + w)   (or y = x when `w` is null) for this rank's `rows` rows, stored
// into EVERY rank's gather buffer at row (my_rank * rows + row).  When the last block has finished, the
// kernel advances a device-resident epoch and writes it into flag slot `my_rank` of every rank's flag
// array; a consumer on rank r waits for flags[src] >= epoch before it reads panel src.  Rows have N
// elements (N % 8 == 0, N <= 8192).  One block handles one row at a time, values stay in registers.
__global__ void __launch_bounds__(COMM_THREADS)
rmsnorm_push_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, PeerTable dst, PeerTable flags, int W,
                    int my_rank, int rows, int N, long long ld_dst, float eps, float offset, float* __restrict__ rstd_out,
                    unsigned long long* __restrict__ epoch_ctr, unsigned int* __restrict__ done_ctr, int* status) {
  __shared__ float sred[COMM_THREADS / 32];
  __shared__ float s_rstd;
  __shared__ unsigned int s_last;
  const int nchunk = N >> 3;
  if (status[0] == 0) {
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      uint4 v[4];
      float sq = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = threadIdx.x + k * COMM_THREADS;
        if (c < nchunk) {
          v[k] = *reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * N + (c << 3));
          if (w != nullptr) {
            const float2 a = unpack_bf16x2(v[k].x), b = unpack_bf16x2(v[k].y), c2 = unpack_bf16x2(v[k].z), d = unpack_bf16x2(v[k].w);
            sq += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c2.x * c2.x + c2.y * c2.y + d.x * d.x + d.y * d.y;
          }
        }
      }
      if (w != nullptr) {
        sq = warp_sum(sq);
        if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = sq;
        __syncthreads();
        if (threadIdx.x < 32) {
          float t = threadIdx.x < COMM_THREADS / 32 ? sred[threadIdx.x] : 0.f;
          t = warp_sum(t);
          if (threadIdx.x == 0) {
            s_rstd = rsqrtf(t / static_cast<float>(N) + eps);
            if (rstd_out != nullptr) rstd_out[row] = s_rstd;
          }
        }
        __syncthreads();
        const float rs = s_rstd;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = threadIdx.x + k * COMM_THREADS;
          if (c < nchunk) {
            const uint4 wu = *reinterpret_cast<const uint4*>(w + (c << 3));
            const float2 a = unpack_bf16x2(v[k].x), b = unpack_bf16x2(v[k].y), c2 = unpack_bf16x2(v[k].z), d = unpack_bf16x2(v[k].w);
            const float2 wa = unpack_bf16x2(wu.x), wb = unpack_bf16x2(wu.y), wc = unpack_bf16x2(wu.z), wd = unpack_bf16x2(wu.w);
            v[k].x = pack_bf16x2(a.x * rs * (offset + wa.x), a.y * rs * (offset + wa.y));
            v[k].y = pack_bf16x2(b.x * rs * (offset + wb.x), b.y * rs * (offset + wb.y));
            v[k].z = pack_bf16x2(c2.x * rs * (offset + wc.x), c2.y * rs * (offset + wc.y));
            v[k].w = pack_bf16x2(d.x * rs * (offset + wd.x), d.y * rs * (offset + wd.y));
          }
        }
      }
      const long long drow = static_cast<long long>(my_rank) * rows + row;
      for (int r = 0; r < W; ++r) {
        bf16* out = static_cast<bf16*>(dst.ptr[(my_rank + r) % W]) + drow * ld_dst;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = threadIdx.x + k * COMM_THREADS;
          if (c < nchunk) *reinterpret_cast<uint4*>(out + (c << 3)) = v[k];
        }
      }
    }
  }
  // completion: every block fences its stores system-wide and takes a ticket; the last one publishes
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(done_ctr, 1u);
    s_last = (ticket == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    __shared__ unsigned long long s_epoch;
    if (threadIdx.x == 0) {
      *done_ctr = 0u;
      s_epoch = *epoch_ctr + 1ull;
      *epoch_ctr = s_epoch;
    }
    __syncthreads();
    if (threadIdx.x < W && status[0] == 0)
      st_release_sys_u64(static_cast<unsigned long long*>(flags.ptr[threadIdx.x]) + my_rank, s_epoch);
  }
}

// out[i] = residual[i] + sum_s stage[s * n + i]  (bf16, fp32 accumulation; n % 8 == 0) — the local half of a
// reduce-scatter whose partial tiles were stored into `stage` by the peers' GEMM epilogues.
__global__ void __launch_bounds__(COMM_THREADS)
reduce_partials_kernel(const bf16* __restrict__ stage, const bf16* __restrict__ residual, bf16* __restrict__ out, int W,
                       long long n, int* status) {
  if (status[0] != 0) return;
  const long long nvec = n >> 3;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual != nullptr) acc_bf16x8(*reinterpret_cast<const uint4*>(residual + (v << 3)), a);
    for (int s = 0; s < W; ++s) acc_bf16x8(*reinterpret_cast<const uint4*>(stage + s * n + (v << 3)), a);
    uint4 o;
    o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
    o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + (v << 3)) = o;
  }
}

__global__ void __launch_bounds__(COMM_THREADS)
allgather_pull_kernel(PeerTable shards, int W, long long n, bf16* __restrict__ out, int* status) {
  if (status[0] != 0) return;
  const long long nvec = n >> 3;
  const long long total = nvec * W;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(v / nvec);
    const long long i = v - r * nvec;
    reinterpret_cast<uint4*>(out)[v] = reinterpret_cast<const uint4*>(shards.ptr[r])[i];
  }
}

// Vocab-parallel cross-entropy combine by peer loads: bufs[r] holds rank r's [2, T] floats
// (log-sum-exp over its vocabulary shard, target logit if the label is in its shard else 0).
__global__ void vp_combine_kernel(PeerTable bufs, int W, int T, float* __restrict__ lse_out, float* __restrict__ tgt_out,
                                  int* status) {
  if (status[0] != 0) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T) return;
  float m = -INFINITY, tg = 0.f;
  float l[MAX_RANKS];
  for (int r = 0; r < W; ++r) {
    const float* b = static_cast<const float*>(bufs.ptr[r]);
    l[r] = b[i];
    tg += b[T + i];
    m = fmaxf(m, l[r]);
  }
  float s = 0.f;
  for (int r = 0; r < W; ++r) s += __expf(l[r] - m);
  lse_out[i] = m + __logf(s);
  tgt_out[i] = tg;
}

}  // namespace cb

namespace {
int comm_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}
int fill_table(cb::PeerTable* t, const unsigned long long* ptrs, int W) {
  if (W < 1 || W > cb::MAX_RANKS) return -1;
  for (int i = 0; i < cb::MAX_RANKS; ++i) t->ptr[i] = i < W ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return 0;
}
}  // namespace

extern "C" {

// Enable loads/stores from kernels on `my_device` to memory of `peer_device` (idempotent).
int cb_enable_peer_access(int my_device, int peer_device) {
  int prev = 0;
  cudaError_t e = cudaGetDevice(&prev);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaSetDevice(my_device);
  if (e != cudaSuccess) return static_cast<int>(e);
  int can = 0;
  e = cudaDeviceCanAccessPeer(&can, my_device, peer_device);
  if (e == cudaSuccess && !can) e = cudaErrorPeerAccessUnsupported;
  if (e == cudaSuccess) {
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      cudaGetLastError();   // clear the sticky-less error state
      e = cudaSuccess;
    }
  }
  cudaSetDevice(prev);
  return static_cast<int>(e);
}

// ---- symmetric allocations and their CUDA IPC handles --------------------------------------------------
// A symmetric buffer is a plain cudaMalloc block on the calling thread's current device.  Its 64-byte IPC
// handle is exchanged on the host; a peer process opens it on ITS current device with lazy peer access, so
// the mapping lives in the opener's own context and no context is ever created on a foreign device.
int cb_symm_alloc(void** out, unsigned long long nbytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, nbytes);
  if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
  e = cudaMemset(p, 0, nbytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { cudaFree(p); return static_cast<int>(e); }
  *out = p;
  return 0;
}

int cb_symm_free(void* p) { return static_cast<int>(cudaFree(p)); }

int cb_ipc_export(void* p, unsigned char* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
  memcpy(handle64, &h, 64);
  return 0;
}

int cb_ipc_open(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
  *out = p;
  return 0;
}

int cb_ipc_close(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

int cb_comm_max_ranks() { return cb::MAX_RANKS; }
int cb_comm_pad_bytes() { return (cb::MAX_RANKS + cb::MAX_RANKS * cb::PAYLOAD_FLOATS / 2) * 8; }
int cb_comm_payload_floats() { return cb::PAYLOAD_FLOATS; }
int cb_comm_grid() { return comm_sms() * 2; }

// pads: host array of W device pointers (each rank's flag pad, cb_comm_pad_bytes() bytes, zeroed once).
int cb_symm_barrier(const unsigned long long* pads, int my_rank, int W, unsigned long long* epoch_ctr,
                    const float* payload_in, float* gathered_out, unsigned long long wait_limit_ns, int* status,
                    void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, pads, W)) return -1;
  cb::symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, my_rank, W, epoch_ctr, payload_in,
                                                                           gathered_out, wait_limit_ns, status);
  return static_cast<int>(cudaGetLastError());
}

// grads: host array of W device pointers to the ranks' bf16 gradient buckets (same layout on every rank).
// partials: cb_comm_grid() floats; payload: cb_comm_payload_floats() floats (receives this rank's sum of squares).
int cb_rs_reduce_sqnorm(const unsigned long long* grads, int W, long long lo, long long hi, float* reduced,
                        float* partials, float* payload, int* status, void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, grads, W) || lo % 8 != 0 || hi % 8 != 0 || hi < lo) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = cb_comm_grid();
  cb::rs_reduce_sqnorm_kernel<<<grid, cb::COMM_THREADS, 0, s>>>(t, W, lo, hi, reduced, partials, status);
  cb::sum_partials_kernel<<<1, 1024, 0, s>>>(partials, grid, payload);
  return static_cast<int>(cudaGetLastError());
}

int cb_adamw_shard_allgather(const unsigned long long* params, int W, int my_rank, long long lo, long long hi,
                             const float* reduced, float* m, float* v, float* master, const unsigned char* chunk_group,
                             const float* hyper, const float* gathered, float max_norm, float* norm_out, int* status,
                             void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, params, W) || lo % 8 != 0 || hi % 8 != 0 || hi < lo) return -1;
  cb::adamw_shard_allgather_kernel<<<cb_comm_grid(), cb::COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      t, W, my_rank, lo, hi, reduced, m, v, master, chunk_group, hyper, gathered, max_norm, norm_out, W, nullptr, status);
  return static_cast<int>(cudaGetLastError());
}

// One bucket of the overlapped reduce-scatter: reduced[0 .. hi - lo) = mean over ranks of grads[r][lo .. hi),
// partials[0 .. grid) = per-block sums of squares.  `grid` blocks of 128 threads (1..1024).
int cb_rs_bucket(const unsigned long long* grads, int W, long long lo, long long hi, float* reduced, float* partials,
                 int grid, int* status, void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, grads, W) || lo % 8 != 0 || hi % 8 != 0 || hi < lo || grid < 1 || grid > 1024) return -1;
  cb::rs_bucket_kernel<<<grid, cb::RSB_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(t, W, lo, hi, reduced, partials,
                                                                                         status);
  return static_cast<int>(cudaGetLastError());
}

// payload[0] = sum(partials[0 .. n)), payload[1..3] = 0 (single block, fixed order).
int cb_sum_partials(const float* partials, int n, float* payload, void* stream) {
  if (n < 1) return -1;
  cb::sum_partials_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(partials, n, payload);
  return static_cast<int>(cudaGetLastError());
}

// AdamW + all-gather for the bucketed layout: this rank's slice has shard_n elements (a multiple of 1024) made of
// one piece per bucket; chunk_off[c] (device, shard_n / 1024 entries) is the offset of chunk c in the flat buffer.
int cb_adamw_shard_allgather_table(const unsigned long long* params, int W, int my_rank, long long shard_n,
                                   const long long* chunk_off, const float* reduced, float* m, float* v, float* master,
                                   const unsigned char* chunk_group, const float* hyper, const float* gathered,
                                   float max_norm, float* norm_out, int* status, void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, params, W) || shard_n <= 0 || shard_n % 1024 != 0 || chunk_off == nullptr) return -1;
  cb::adamw_shard_allgather_kernel<<<cb_comm_grid(), cb::COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      t, W, my_rank, 0, shard_n, reduced, m, v, master, chunk_group, hyper, gathered, max_norm, norm_out, W, chunk_off,
      status);
  return static_cast<int>(cudaGetLastError());
}

// ZeRO-3 flavour of the update: parameters stay sharded, so the new bf16 values are written only to this
// rank's shard (`shard`, n elements, n % 1024 == 0); the clip coefficient still comes from all W ranks'
// norm shares in `gathered`.
int cb_adamw_shard_local(void* shard, int W, long long n, const float* reduced, float* m, float* v, float* master,
                         const unsigned char* chunk_group, const float* hyper, const float* gathered, float max_norm,
                         float* norm_out, int* status, void* stream) {
  if (n <= 0 || n % 8 != 0 || W < 1 || W > cb::MAX_RANKS) return -1;
  cb::PeerTable t;
  for (int i = 0; i < cb::MAX_RANKS; ++i) t.ptr[i] = nullptr;
  t.ptr[0] = shard;
  cb::adamw_shard_allgather_kernel<<<cb_comm_grid(), cb::COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      t, W, 0, 0, n, reduced, m, v, master, chunk_group, hyper, gathered, max_norm, norm_out, 1, nullptr, status);
  return static_cast<int>(cudaGetLastError());
}

// Parameter all-gather by pull: out[r * n + i] = shards[r][i] (bf16, n % 8 == 0).  Shards only change in
// the optimizer step (followed by a barrier), so no flag is needed while a step's forward/backward read them.
int cb_allgather_pull(const unsigned long long* shards, int W, long long n, void* out, int* status, void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, shards, W) || n <= 0 || n % 8 != 0) return -1;
  cb::allgather_pull_kernel<<<cb_comm_grid(), cb::COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      t, W, n, static_cast<cb::bf16*>(out), status);
  return static_cast<int>(cudaGetLastError());
}

int cb_allreduce_pull(const unsigned long long* bufs, int W, long long n, float scale, void* out, int* status,
                      void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, bufs, W) || n % 8 != 0) return -1;
  cb::allreduce_pull_kernel<<<cb_comm_grid(), cb::COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      t, W, n, scale, static_cast<cb::bf16*>(out), status);
  return static_cast<int>(cudaGetLastError());
}


// Tensor/sequence parallel push all-gather (optionally fused with RMSNorm when w != null).
// dst / flags: host arrays of W device addresses (every rank's gather buffer and flag array).
int cb_rmsnorm_push(const void* x, const void* w, const unsigned long long* dst, const unsigned long long* flags, int W,
                    int my_rank, int rows, int N, long long ld_dst, float eps, float offset, float* rstd_out,
                    unsigned long long* epoch_ctr, unsigned int* done_ctr, int* status, void* stream) {
  if (rows <= 0 || N <= 0 || N % 8 != 0 || N > 8 * 4 * cb::COMM_THREADS || ld_dst % 8 != 0) return -1;
  cb::PeerTable d, f;
  if (fill_table(&d, dst, W) || fill_table(&f, flags, W)) return -2;
  int grid = comm_sms() * 4;
  if (grid > rows) grid = rows;
  cb::rmsnorm_push_kernel<<<grid, cb::COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const cb::bf16*>(x), static_cast<const cb::bf16*>(w), d, f, W, my_rank, rows, N, ld_dst, eps, offset,
      rstd_out, epoch_ctr, done_ctr, status);
  return static_cast<int>(cudaGetLastError());
}

int cb_reduce_partials(const void* stage, const void* residual, void* out, int W, long long n, int* status, void* stream) {
  if (n <= 0 || n % 8 != 0 || W < 1) return -1;
  long long blocks = (n / 8 + cb::COMM_THREADS - 1) / cb::COMM_THREADS;
  const long long cap = static_cast<long long>(comm_sms()) * 8;
  if (blocks > cap) blocks = cap;
  cb::reduce_partials_kernel<<<static_cast<int>(blocks), cb::COMM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const cb::bf16*>(stage), static_cast<const cb::bf16*>(residual), static_cast<cb::bf16*>(out), W, n, status);
  return static_cast<int>(cudaGetLastError());
}

int cb_vp_combine(const unsigned long long* bufs, int W, int T, float* lse_out, float* tgt_out, int* status, void* stream) {
  cb::PeerTable t;
  if (fill_table(&t, bufs, W) || T <= 0) return -1;
  cb::vp_combine_kernel<<<(T + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(t, W, T, lse_out, tgt_out, status);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
