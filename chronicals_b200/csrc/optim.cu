// Multi-tensor optimizer kernels: one launch updates every parameter tensor.
//
// The tensor table (pointers, sizes, group ids) lives in device memory and is
// uploaded once, because parameter addresses never change; per-group
// hyper-parameters (learning rate, weight decay, betas, bias corrections) live
// in a small device array refreshed by an async copy each step, and the clip
// coefficient is read from a device scalar - so a whole step needs no host
// synchronisation and can be replayed from a CUDA graph.
//
// Replaces the reference's one-Triton-launch-per-tensor AdamW
// (chronicals/optimizers/fused_adamw.py:45-101, :390-423) and its
// torch._foreach_norm based clipping (:169-219).
#include "common.cuh"

namespace cb {

constexpr int OPT_THREADS = 256;
constexpr int OPT_CHUNK = 8192;   // elements per block

struct TensorTable {
  void* const* p;          // parameter (bf16 or fp32)
  const void* const* g;    // gradient, same dtype as the parameter
  float* const* m;
  float* const* v;
  float* const* master;    // fp32 master copy, entries may be null
  const long long* numel;
  const int* group;        // index into the hyper-parameter table
  const int* chunk_start;  // [n_tensors + 1] prefix sum of chunk counts
  int n_tensors;
};

// hyper[group * 8 + ...]: lr, weight_decay, beta1, beta2, eps, bias_corr1, bias_corr2, unused
constexpr int HYPER_STRIDE = 8;

__device__ __forceinline__ int find_tensor(const int* chunk_start, int n, int chunk) {
  int lo = 0, hi = n;  // chunk_start[lo] <= chunk < chunk_start[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (chunk_start[mid] <= chunk) lo = mid;
    else hi = mid;
  }
  return lo;
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16(v); }

// AdamW in the reference's order: g *= clip; p *= 1 - lr*wd; m, v EMAs; p -= lr/bc1 * m / (sqrt(v/bc2) + eps)
template <typename T>
__global__ void __launch_bounds__(OPT_THREADS)
adamw_multi_kernel(TensorTable tt, const float* __restrict__ hyper, const float* __restrict__ clip_coef) {
  const int ti = find_tensor(tt.chunk_start, tt.n_tensors, blockIdx.x);
  const long long off = static_cast<long long>(blockIdx.x - tt.chunk_start[ti]) * OPT_CHUNK;
  const long long n = tt.numel[ti];
  const float* h = hyper + tt.group[ti] * HYPER_STRIDE;
  const float lr = h[0], wd = h[1], b1 = h[2], b2 = h[3], eps = h[4], bc1 = h[5], bc2 = h[6];
  const float clip = clip_coef ? clip_coef[0] : 1.f;
  T* p = static_cast<T*>(tt.p[ti]);
  const T* g = static_cast<const T*>(tt.g[ti]);
  float* m = tt.m[ti];
  float* v = tt.v[ti];
  float* master = tt.master ? tt.master[ti] : nullptr;
  const float step_size = lr / bc1;
  const float inv_bc2 = 1.f / bc2;
  const float decay = 1.f - lr * wd;
  const long long end = (off + OPT_CHUNK < n) ? off + OPT_CHUNK : n;
  constexpr int VEC = 4;
  const bool aligned = (reinterpret_cast<uintptr_t>(p) % (VEC * sizeof(T)) == 0) &&
                       (reinterpret_cast<uintptr_t>(g) % (VEC * sizeof(T)) == 0) &&
                       (reinterpret_cast<uintptr_t>(m) % 16 == 0) && (reinterpret_cast<uintptr_t>(v) % 16 == 0) &&
                       (master == nullptr || reinterpret_cast<uintptr_t>(master) % 16 == 0);
  if (aligned) {
    for (long long i = off + threadIdx.x * VEC; i < end; i += OPT_THREADS * VEC) {
      if (i + VEC <= end) {
        float pf[VEC], gf[VEC];
        if (sizeof(T) == 2) {
          const uint2 pu = *reinterpret_cast<const uint2*>(p + i);
          const uint2 gu = *reinterpret_cast<const uint2*>(g + i);
          const float2 p0 = unpack_bf16x2(pu.x), p1 = unpack_bf16x2(pu.y);
          const float2 g0 = unpack_bf16x2(gu.x), g1 = unpack_bf16x2(gu.y);
          pf[0] = p0.x; pf[1] = p0.y; pf[2] = p1.x; pf[3] = p1.y;
          gf[0] = g0.x; gf[1] = g0.y; gf[2] = g1.x; gf[3] = g1.y;
        } else {
          const float4 pu = *reinterpret_cast<const float4*>(p + i);
          const float4 gu = *reinterpret_cast<const float4*>(g + i);
          pf[0] = pu.x; pf[1] = pu.y; pf[2] = pu.z; pf[3] = pu.w;
          gf[0] = gu.x; gf[1] = gu.y; gf[2] = gu.z; gf[3] = gu.w;
        }
        float4 mv = *reinterpret_cast<const float4*>(m + i);
        float4 vv = *reinterpret_cast<const float4*>(v + i);
        float mf[VEC] = {mv.x, mv.y, mv.z, mv.w};
        float vf[VEC] = {vv.x, vv.y, vv.z, vv.w};
        if (master) {
          const float4 w = *reinterpret_cast<const float4*>(master + i);
          pf[0] = w.x; pf[1] = w.y; pf[2] = w.z; pf[3] = w.w;
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const float gj = gf[j] * clip;
          float w = pf[j] * decay;
          mf[j] = b1 * mf[j] + (1.f - b1) * gj;
          vf[j] = b2 * vf[j] + (1.f - b2) * gj * gj;
          w -= step_size * mf[j] / (sqrtf(vf[j] * inv_bc2) + eps);
          pf[j] = w;
        }
        *reinterpret_cast<float4*>(m + i) = make_float4(mf[0], mf[1], mf[2], mf[3]);
        *reinterpret_cast<float4*>(v + i) = make_float4(vf[0], vf[1], vf[2], vf[3]);
        if (master) *reinterpret_cast<float4*>(master + i) = make_float4(pf[0], pf[1], pf[2], pf[3]);
        if (sizeof(T) == 2) {
          uint2 o;
          o.x = pack_bf16x2(pf[0], pf[1]);
          o.y = pack_bf16x2(pf[2], pf[3]);
          *reinterpret_cast<uint2*>(p + i) = o;
        } else {
          *reinterpret_cast<float4*>(p + i) = make_float4(pf[0], pf[1], pf[2], pf[3]);
        }
      } else {
        for (long long k = i; k < end; ++k) {
          const float gj = to_f<T>(g[k]) * clip;
          float w = (master ? master[k] : to_f<T>(p[k])) * decay;
          const float mj = b1 * m[k] + (1.f - b1) * gj;
          const float vj = b2 * v[k] + (1.f - b2) * gj * gj;
          w -= step_size * mj / (sqrtf(vj * inv_bc2) + eps);
          m[k] = mj; v[k] = vj;
          if (master) master[k] = w;
          p[k] = from_f<T>(w);
        }
      }
    }
  } else {
    for (long long k = off + threadIdx.x; k < end; k += OPT_THREADS) {
      const float gj = to_f<T>(g[k]) * clip;
      float w = (master ? master[k] : to_f<T>(p[k])) * decay;
      const float mj = b1 * m[k] + (1.f - b1) * gj;
      const float vj = b2 * v[k] + (1.f - b2) * gj * gj;
      w -= step_size * mj / (sqrtf(vj * inv_bc2) + eps);
      m[k] = mj; v[k] = vj;
      if (master) master[k] = w;
      p[k] = from_f<T>(w);
    }
  }
}

// sum of squares of every gradient: one partial per chunk (deterministic), reduced by sqnorm_finalize_kernel
template <typename T>
__global__ void __launch_bounds__(OPT_THREADS)
grad_sqnorm_kernel(TensorTable tt, float* __restrict__ partials) {
  __shared__ float sred[OPT_THREADS / 32];
  const int ti = find_tensor(tt.chunk_start, tt.n_tensors, blockIdx.x);
  const long long off = static_cast<long long>(blockIdx.x - tt.chunk_start[ti]) * OPT_CHUNK;
  const long long n = tt.numel[ti];
  const T* g = static_cast<const T*>(tt.g[ti]);
  const long long end = (off + OPT_CHUNK < n) ? off + OPT_CHUNK : n;
  float s = 0.f;
  if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(g) % 16 == 0)) {
    for (long long i = off + threadIdx.x * 8; i < end; i += OPT_THREADS * 8) {
      if (i + 8 <= end) {
        const uint4 u = *reinterpret_cast<const uint4*>(g + i);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        s += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
      } else {
        for (long long k = i; k < end; ++k) { const float f = to_f<T>(g[k]); s += f * f; }
      }
    }
  } else {
    for (long long k = off + threadIdx.x; k < end; k += OPT_THREADS) { const float f = to_f<T>(g[k]); s += f * f; }
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < OPT_THREADS / 32 ? sred[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
}

// out[0] = sum of partials (+ extra_sq[0], e.g. other ranks' share), out[1] = norm,
// out[2] = clip coefficient min(1, max_norm / (norm + 1e-6)); max_norm <= 0 disables clipping.
__global__ void __launch_bounds__(1024)
sqnorm_finalize_kernel(const float* __restrict__ partials, int n, const float* __restrict__ extra_sq, float max_norm,
                       float* __restrict__ out) {
  __shared__ double sred[32];
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += static_cast<double>(partials[i]);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += sred[i];
    if (extra_sq) t += static_cast<double>(extra_sq[0]);
    const float norm = static_cast<float>(sqrt(t));
    out[0] = static_cast<float>(t);
    out[1] = norm;
    out[2] = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  }
}


// ------------------------------------------------------------------------------------------------------
// AdamW with 8-bit block-quantised moments (blocks of 256 elements, one fp32 absmax per block; the first
// moment in a signed linear code q = round(m / absmax * 127), the square root of the second moment in an
// unsigned code q = round(sqrt(v) / absmax * 255)).  One warp owns one block: dequantise, update in fp32,
// find the new absmax with shuffles, re-quantise, store.  10 bytes of traffic per parameter instead of 18.
// Replaces the reference's bitsandbytes wrappers (chronicals/optimizers/optimizers_8bit.py:117-336).
template <typename T>
__global__ void __launch_bounds__(256)
adamw8bit_kernel(T* __restrict__ p, const T* __restrict__ g, signed char* __restrict__ mq, unsigned char* __restrict__ vq,
                 float* __restrict__ m_absmax, float* __restrict__ v_absmax, long long n, float lr, float beta1,
                 float beta2, float eps, float weight_decay, float bc1, float bc2) {
  const long long nblk = (n + 255) / 256;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const float step = lr / bc1, inv_bc2 = 1.f / bc2, decay = 1.f - lr * weight_decay;
  for (long long b = warp0; b < nblk; b += nwarps) {
    const float am = m_absmax[b] * (1.f / 127.f), av = v_absmax[b] * (1.f / 255.f);
    float m[8], rv[8];
    float mx_m = 0.f, mx_v = 0.f;
    const long long base = b * 256 + lane * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = base + j;
      m[j] = 0.f;
      rv[j] = 0.f;
      if (i < n) {
        const float gi = static_cast<float>(g[i]);
        const float sv = static_cast<float>(vq[i]) * av;          // sqrt(v)
        const float mi = beta1 * (static_cast<float>(mq[i]) * am) + (1.f - beta1) * gi;
        const float vi = beta2 * sv * sv + (1.f - beta2) * gi * gi;
        float x = static_cast<float>(p[i]) * decay;
        x -= step * mi / (sqrtf(vi * inv_bc2) + eps);
        p[i] = static_cast<T>(x);
        m[j] = mi;
        rv[j] = sqrtf(vi);
        mx_m = fmaxf(mx_m, fabsf(mi));
        mx_v = fmaxf(mx_v, rv[j]);
      }
    }
    mx_m = fmaxf(warp_max(mx_m), 1e-30f);
    mx_v = fmaxf(warp_max(mx_v), 1e-30f);
    if (lane == 0) {
      m_absmax[b] = mx_m;
      v_absmax[b] = mx_v;
    }
    const float sm = 127.f / mx_m, sv2 = 255.f / mx_v;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = base + j;
      if (i < n) {
        mq[i] = static_cast<signed char>(fminf(fmaxf(rintf(m[j] * sm), -127.f), 127.f));
        vq[i] = static_cast<unsigned char>(fminf(fmaxf(rintf(rv[j] * sv2), 0.f), 255.f));
      }
    }
  }
}

}  // namespace cb

extern "C" {

int cb_opt_chunk() { return cb::OPT_CHUNK; }

// The table arrays are device pointers (see TensorTable); total_chunks = chunk_start[n_tensors].
int cb_adamw_multi(void* const* p, const void* const* g, float* const* m, float* const* v, float* const* master,
                   const long long* numel, const int* group, const int* chunk_start, int n_tensors, int total_chunks,
                   const float* hyper, const float* clip_coef, int is_bf16, void* stream) {
  if (n_tensors <= 0 || total_chunks <= 0) return -1;
  cb::TensorTable tt = {p, g, m, v, master, numel, group, chunk_start, n_tensors};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16) cb::adamw_multi_kernel<cb::bf16><<<total_chunks, cb::OPT_THREADS, 0, s>>>(tt, hyper, clip_coef);
  else cb::adamw_multi_kernel<float><<<total_chunks, cb::OPT_THREADS, 0, s>>>(tt, hyper, clip_coef);
  return static_cast<int>(cudaGetLastError());
}

// partials: scratch of total_chunks floats; out: 3 floats (sum of squares, norm, clip coefficient).
int cb_grad_clip_coef(const void* const* g, const long long* numel, const int* chunk_start, int n_tensors,
                      int total_chunks, float* partials, const float* extra_sq, float max_norm, float* out,
                      int is_bf16, void* stream) {
  if (n_tensors <= 0 || total_chunks <= 0) return -1;
  cb::TensorTable tt = {nullptr, g, nullptr, nullptr, nullptr, numel, nullptr, chunk_start, n_tensors};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16) cb::grad_sqnorm_kernel<cb::bf16><<<total_chunks, cb::OPT_THREADS, 0, s>>>(tt, partials);
  else cb::grad_sqnorm_kernel<float><<<total_chunks, cb::OPT_THREADS, 0, s>>>(tt, partials);
  cb::sqnorm_finalize_kernel<<<1, 1024, 0, s>>>(partials, total_chunks, extra_sq, max_norm, out);
  return static_cast<int>(cudaGetLastError());
}


// 8-bit AdamW step on one tensor.  is_bf16 selects the parameter / gradient dtype (bf16 or fp32).
int cb_adamw8bit(void* p, const void* g, void* mq, void* vq, float* m_absmax, float* v_absmax, long long n, int is_bf16,
                 float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2, void* stream) {
  if (n <= 0) return -1;
  const long long nblk = (n + 255) / 256;
  long long blocks = (nblk + 7) / 8;                      // 8 warps (quantisation blocks) per CTA
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (blocks > static_cast<long long>(sms) * 8) blocks = static_cast<long long>(sms) * 8;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    cb::adamw8bit_kernel<cb::bf16><<<static_cast<int>(blocks), 256, 0, s>>>(
        static_cast<cb::bf16*>(p), static_cast<const cb::bf16*>(g), static_cast<signed char*>(mq),
        static_cast<unsigned char*>(vq), m_absmax, v_absmax, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2);
  else
    cb::adamw8bit_kernel<float><<<static_cast<int>(blocks), 256, 0, s>>>(
        static_cast<float*>(p), static_cast<const float*>(g), static_cast<signed char*>(mq),
        static_cast<unsigned char*>(vq), m_absmax, v_absmax, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
