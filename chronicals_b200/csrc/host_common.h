// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda) and the SM count.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

namespace cbhost {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D tensor map over this GPU's own memory: `inner` contiguous elements per row, `outer` rows,
// row pitch `ld` elements, 128-byte swizzle, out-of-range reads return zero.
inline int make_tmap(CUtensorMap* out, const void* base, unsigned long long inner, unsigned long long outer,
                     unsigned long long ld, unsigned box_inner, unsigned box_outer, int elem_bytes = 2) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -10;
  // The driver call needs a context bound to the calling thread.  A thread that has not used this
  // library's CUDA runtime yet (an autograd worker, say) may have none: bind the primary context once.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * elem_bytes) % 16 != 0) return -11;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    // A thread that has not yet touched this library's CUDA runtime (e.g. an autograd worker)
    // may have no context bound for it: bind the primary context and try once more.
    const int first = static_cast<int>(r);
    cudaFree(nullptr);
    r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
      if (getenv("CB_DEBUG_TMAP")) fprintf(stderr, "[chronicals_b200] tensor-map encode succeeded on retry (first CUresult %d)\n", first);
      return 0;
    }
    fprintf(stderr, "[chronicals_b200] cuTensorMapEncodeTiled failed: CUresult %d base %p inner %llu outer %llu ld %llu "
            "box %u x %u elem %d\n", static_cast<int>(r), base, inner, outer, ld, box_inner, box_outer, elem_bytes);
    return -12;
  }
  return 0;
}

inline int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace cbhost
