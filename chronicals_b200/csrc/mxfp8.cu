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
                   bf16* __restrict__ deq, long long M, int K, long long ldx, int packed_kb4, int tile_rows) {
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
    // (rows grouped in tiles of `tile_rows`, each tile padded to a multiple of 128 rows: mp is the padded row)
    long long sidx = m * nblk + kb;
    if (packed_kb4 > 0) {
      const long long tile = m / tile_rows;
      const long long mp = tile * ((tile_rows + 127) / 128 * 128) + (m - tile * tile_rows);
      sidx = ((mp >> 7) * packed_kb4 + (kb >> 2)) * 512 + (mp & 31) * 16 + ((mp >> 5) & 3) * 4 + (kb & 3);
    }
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


// e8m0 exponent e with 2^e >= amax / fmt_max (exact: taken from the float's own exponent and mantissa)
__device__ __forceinline__ int mx_scale_exp(float amax, float fmt_max) {
  if (!(amax > 0.f)) return -127;
  int ex;
  const float mant = frexpf(amax / fmt_max, &ex);      // ratio = mant * 2^ex, mant in [0.5, 1)
  const int e = (mant == 0.5f) ? ex - 1 : ex;
  return max(-127, min(127, e));
}
// byte index of the scale of (row, block kb) in the packed atoms (rows grouped in tiles of tile_rows)
__device__ __forceinline__ long long mx_sf_index(long long row, int kb, int kb4, int tile_rows) {
  const long long tile = row / tile_rows;
  const long long mp = tile * ((tile_rows + 127) / 128 * 128) + (row - tile * tile_rows);
  return ((mp >> 7) * kb4 + (kb >> 2)) * 512 + (mp & 31) * 16 + ((mp >> 5) & 3) * 4 + (kb & 3);
}

// MXFP8 copy of the TRANSPOSE of x [R, C] (bf16): q_col [C, R] with blocks of 32 along R (the dimension a
// gradient GEMM contracts over) and packed scales for rows c, without materialising a bf16 transpose.
// A block owns 32 rows x 256 columns; thread t owns column c0 + t, keeps its 32 values (one whole scale
// block) in registers, and writes them as 32 contiguous bytes of row c of the output.
template <int E5M2>
__global__ void __launch_bounds__(256)
mxfp8_quant_transposed_kernel(const bf16* __restrict__ x, long long R, int C, long long ldx,
                              unsigned char* __restrict__ q_col, unsigned char* __restrict__ sf_col, int col_tile) {
  const float fmt_max = E5M2 ? 57344.f : 448.f;
  const long long r0 = static_cast<long long>(blockIdx.y) * 32;
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  float v[32];
#pragma unroll
  for (int r = 0; r < 32; ++r) v[r] = __bfloat162float(x[(r0 + r) * ldx + c]);
  float amax = 0.f;
#pragma unroll
  for (int r = 0; r < 32; ++r) amax = fmaxf(amax, fabsf(v[r]));
  const int e = mx_scale_exp(amax, fmt_max);
  const float inv = exp2f(static_cast<float>(-e));
  sf_col[mx_sf_index(c, static_cast<int>(r0 >> 5), static_cast<int>((R + 127) / 128), col_tile)] =
      static_cast<unsigned char>(e + 127);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_fp8x2_storage_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i] * inv, v[4 * i + 1] * inv),
                                                             __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
    const __nv_fp8x2_storage_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv),
                                                             __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
    w[i] = static_cast<uint32_t>(p0) | (static_cast<uint32_t>(p1) << 16);
  }
  uint4* dst = reinterpret_cast<uint4*>(q_col + static_cast<long long>(c) * R + r0);
  dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
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
        static_cast<cb::bf16*>(deq), M, K, ldx, 0, 128);
  else
    cb::mxfp8_quant_kernel<0><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), static_cast<unsigned char*>(scales),
        static_cast<cb::bf16*>(deq), M, K, ldx, 0, 128);
  return static_cast<int>(cudaGetLastError());
}


// As cb_mxfp8_quant, but the scales go into the packed atoms of the block-scaled GEMM.  Rows are grouped in
// tiles of `tile_rows` (128 for the A operand and for the single-CTA kernel, the pair kernel's B tile otherwise),
// each tile padded to a multiple of 128 rows: `sf` has tiles * ceil(tile_rows/128) * ceil(K/128) * 512 bytes and
// must have been filled with a finite scale (127) beforehand wherever padding exists, since bytes of rows and
// blocks outside the matrix are not written.
int cb_mxfp8_quant_packed(const void* x, void* q, void* sf, long long M, int K, long long ldx, int e5m2, int tile_rows,
                          void* stream) {
  if (M <= 0 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || tile_rows <= 0 || tile_rows % 32 != 0) return -1;
  long long blocks = (M * (K / 32) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int kb4 = (K + 127) / 128;
  if (e5m2)
    cb::mxfp8_quant_kernel<1><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), static_cast<unsigned char*>(sf), nullptr, M, K,
        ldx, kb4, tile_rows);
  else
    cb::mxfp8_quant_kernel<0><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        static_cast<const cb::bf16*>(x), static_cast<unsigned char*>(q), static_cast<unsigned char*>(sf), nullptr, M, K,
        ldx, kb4, tile_rows);
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

// x [R, C] bf16 (pitch ldx) -> q_col [C, R] = MXFP8 copy of the transpose, packed scales along R for rows c
// (col_tile as tile_rows in cb_mxfp8_quant_packed; the scale buffer pre-filled with 127 where padding exists).
// R a multiple of 32.
int cb_mxfp8_quant_transposed(const void* x, long long R, int C, long long ldx, void* q_col, void* sf_col, int col_tile,
                              int e5m2, void* stream) {
  if (R <= 0 || C <= 0 || R % 32 != 0 || col_tile <= 0 || col_tile % 32 != 0 || q_col == nullptr || sf_col == nullptr)
    return -1;
  if (R / 32 > 65535) return -2;
  const dim3 grid(static_cast<unsigned>((C + 255) / 256), static_cast<unsigned>(R / 32));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e5m2)
    cb::mxfp8_quant_transposed_kernel<1><<<grid, 256, 0, s>>>(static_cast<const cb::bf16*>(x), R, C, ldx,
        static_cast<unsigned char*>(q_col), static_cast<unsigned char*>(sf_col), col_tile);
  else
    cb::mxfp8_quant_transposed_kernel<0><<<grid, 256, 0, s>>>(static_cast<const cb::bf16*>(x), R, C, ldx,
        static_cast<unsigned char*>(q_col), static_cast<unsigned char*>(sf_col), col_tile);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
