// MXFP8 (OCP microscaling) quantisation: 32-element blocks along the last dimension, one e8m0
// (power-of-two) scale per block, elements in e4m3 or e5m2.
//
//   scale = 2^ceil(log2(amax / fmt_max))     (so amax / scale <= fmt_max; zero blocks get 2^-127)
//   q     = round_to_nearest_even_saturating(x / scale)
//
// One warp handles one row segment of 32 blocks at a time: each lane owns one block (32 contiguous
// bf16 = 64 bytes), so the block maximum needs no shuffles.  Optionally also writes the exactly
// dequantised bf16 values (an e4m3 value times a power of two is representable in bf16), which is
// what the bf16 tensor-core GEMM consumes when a block-scaled result is wanted.
//
// Replaces the reference's simulated 128-block quantisers (chronicals/utils/fp8_deepseek.py:512-610,
// fake rounding floor(x*8+.5)/8) with real hardware conversions and MX scaling.
#include "common.cuh"

#include <cuda_fp8.h>

namespace cb {

template <int E5M2>
__global__ void __launch_bounds__(256)
mxfp8_quant_kernel(const bf16* __restrict__ x, unsigned char* __restrict__ q, unsigned char* __restrict__ scales,
                   bf16* __restrict__ deq, long long M, int K, long long ldx, int packed_kb4) {
  const int nblk = K / 32;
  const long long total = M * nblk;
  const float fmt_max = E5M2 ? 57344.f : 448.f;
  for (long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; b < total;
       b += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = b / nblk;
    const int kb = static_cast<int>(b % nblk);
    const uint4* src = reinterpret_cast<const uint4*>(x + m * ldx + kb * 32);
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = src[i];
      const float2 a = unpack_bf16x2(u.x), c = unpack_bf16x2(u.y), d = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
      v[8 * i + 0] = a.x; v[8 * i + 1] = a.y; v[8 * i + 2] = c.x; v[8 * i + 3] = c.y;
      v[8 * i + 4] = d.x; v[8 * i + 5] = d.y; v[8 * i + 6] = e.x; v[8 * i + 7] = e.y;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    // exponent e with 2^e >= amax / fmt_max, exact via the float's own exponent and mantissa
    int e = -127;
    if (amax > 0.f) {
      const float ratio = amax / fmt_max;
      int ex;
      const float mant = frexpf(ratio, &ex);          // ratio = mant * 2^ex, mant in [0.5, 1)
      e = (mant == 0.5f) ? ex - 1 : ex;
      e = max(-127, min(127, e));
    }
    const float inv = exp2f(static_cast<float>(-e));
    const float sc = exp2f(static_cast<float>(e));
    // packed_kb4 > 0: the 512-byte atoms ([128 rows][4 blocks], byte (r%32)*16 + (r/32%4)*4 + kb%4) that the
    // block-scaled tensor-core GEMM copies to tensor memory as they are
    const long long sidx = packed_kb4 > 0
        ? ((m >> 7) * packed_kb4 + (kb >> 2)) * 512 + (m & 31) * 16 + ((m >> 5) & 3) * 4 + (kb & 3)
        : m * nblk + kb;
    scales[sidx] = static_cast<unsigned char>(e + 127);
    unsigned char out[32];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const float2 pr = make_float2(v[i] * inv, v[i + 1] * inv);
      const __nv_fp8x2_storage_t p = __nv_cvt_float2_to_fp8x2(pr, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
      out[i] = static_cast<unsigned char>(p & 0xff);
      out[i + 1] = static_cast<unsigned char>(p >> 8);
    }
    uint4* dq = reinterpret_cast<uint4*>(q + m * K + kb * 32);
    dq[0] = *reinterpret_cast<uint4*>(&out[0]);
    dq[1] = *reinterpret_cast<uint4*>(&out[16]);
    if (deq != nullptr) {
      float w[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const __half_raw hr = __nv_cvt_fp8_to_halfraw(out[i], E5M2 ? __NV_E5M2 : __NV_E4M3);
        w[i] = __half2float(*reinterpret_cast<const __half*>(&hr)) * sc;
      }
      uint4* dd = reinterpret_cast<uint4*>(deq + m * K + kb * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 u;
        u.x = pack_bf16x2(w[8 * i + 0], w[8 * i + 1]); u.y = pack_bf16x2(w[8 * i + 2], w[8 * i + 3]);
        u.z = pack_bf16x2(w[8 * i + 4], w[8 * i + 5]); u.w = pack_bf16x2(w[8 * i + 6], w[8 * i + 7]);
        dd[i] = u;
      }
    }
  }
}


// Row-wise e4m3 quantisation for the FP8 tensor-core GEMM: scale[row] = amax(row) / 448 (fp32),
// q[row, k] = e4m3(x[row, k] / scale[row]).  One warp per row, 16-byte loads, 8-byte stores.
__global__ void __launch_bounds__(256)
rowquant_e4m3_kernel(const bf16* __restrict__ x, unsigned char* __restrict__ q, float* __restrict__ scale, long long M,
                     int K, long long ldx, long long ldq) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int nvec = K >> 3;
  for (long long row = warp0; row < M; row += nwarps) {
    const bf16* xr = x + row * ldx;
    float amax = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + (v << 3));
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                               fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y)))));
    }
    amax = warp_max(amax);
    const float sc = fmaxf(amax, 1e-30f) * (1.f / 448.f);
    const float inv = 1.f / sc;
    if (lane == 0) scale[row] = sc;
    unsigned char* qr = q + row * ldq;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + (v << 3));
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
      unsigned long long packed = 0ull;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const unsigned long long byte = __nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3);
        packed |= byte << (8 * j);
      }
      *reinterpret_cast<unsigned long long*>(qr + (v << 3)) = packed;
    }
  }
}

}  // namespace cb

extern "C" {

// x: bf16 [M, K] with row pitch ldx (K a multiple of 32, ldx a multiple of 8); q: uint8 [M, K] fp8 bit
// patterns; scales: uint8 [M, K/32] biased exponents; deq: bf16 [M, K] or null.
int cb_mxfp8_quant(const void* x, void* q, void* scales, void* deq, long long M, int K, long long ldx, int e5m2,
                   void* stream) {
  if (M <= 0 || K <= 0 || K % 32 != 0 || ldx % 8 != 0) return -1;
  long long blocks = (M * (K / 32) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e5m2)
    cb::mxfp8_quant_kernel<1><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), static_cast<unsigned char*>(scales),
        static_cast<cb::bf16*>(deq), M, K, ldx, 0);
  else
    cb::mxfp8_quant_kernel<0><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), static_cast<unsigned char*>(scales),
        static_cast<cb::bf16*>(deq), M, K, ldx, 0);
  return static_cast<int>(cudaGetLastError());
}


// As cb_mxfp8_quant, but the scales go into the packed atoms of the block-scaled GEMM: `sf` has
// ceil(M/128) * ceil(K/128) * 512 bytes and must have been filled with a finite scale (127) beforehand where
// M or K/32 is not a multiple of 128 or 4, since bytes of rows and blocks outside the matrix are not written.
int cb_mxfp8_quant_packed(const void* x, void* q, void* sf, long long M, int K, long long ldx, int e5m2, void* stream) {
  if (M <= 0 || K <= 0 || K % 32 != 0 || ldx % 8 != 0) return -1;
  long long blocks = (M * (K / 32) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int kb4 = (K + 127) / 128;
  if (e5m2)
    cb::mxfp8_quant_kernel<1><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), static_cast<unsigned char*>(sf), nullptr, M, K,
        ldx, kb4);
  else
    cb::mxfp8_quant_kernel<0><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), static_cast<unsigned char*>(sf), nullptr, M, K,
        ldx, kb4);
  return static_cast<int>(cudaGetLastError());
}


// x: bf16 [M, K] (pitch ldx elements, K a multiple of 16); q: e4m3 bytes [M, K] (pitch ldq bytes, multiple of 16);
// scale: fp32 [M].
int cb_rowquant_e4m3(const void* x, void* q, float* scale, long long M, int K, long long ldx, long long ldq, void* stream) {
  if (M <= 0 || K <= 0 || K % 16 != 0 || ldx % 8 != 0 || ldq % 16 != 0) return -1;
  long long blocks = (M + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cb::rowquant_e4m3_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), scale, M, K, ldx, ldq);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
