/* Allocation-free entry point of the chronicals_b200 kernel library.
 *
 * This has no counterpart in the reference project; it exists for hosts of this library that
 * are not allowed to allocate device memory at the point where they call in.  Examples: code
 * running inside a memory-planned region where every byte was reserved up front, a plugin
 * called from someone else's runtime that owns the allocator, or a real-time control loop in
 * which a cudaMalloc (which may synchronise the whole device) is not acceptable.
 *
 * cb_rmsnorm_bwd_noalloc computes the same thing as cb_rmsnorm_bwd:
 *
 *     xhat = h * rstd,  g = dy * (w + offset)
 *     dx   = rstd * (g - xhat * mean(g * xhat))  (+ dres_in)
 *     dw   = sum over rows of dy * xhat          (+ dw when accumulate_dw != 0)
 *
 * but it needs no scratch buffer from the caller and calls no cudaMalloc / cudaFree or any
 * other allocating routine: the per-block partial sums of dw are kept in a fixed array that is
 * part of the library image.  The caller still provides every input and output:
 *
 *     dy, h     bf16 [M, N] row-major            rstd  fp32 [M]
 *     w         bf16 [N]                         dres_in  bf16 [M, N] or NULL
 *     dx        bf16 [M, N] (out)                dw    bf16 [N] (out) or NULL
 *
 * Limits and rules
 *   - N must be a multiple of 8 and at most CB_NOALLOC_RMSNORM_MAX_N; larger N returns -2 and
 *     nothing is launched (use cb_rmsnorm_bwd with your own scratch instead).  M is unlimited.
 *   - The built-in array is CB_NOALLOC_RMSNORM_MAX_BLOCKS * CB_NOALLOC_RMSNORM_MAX_N floats
 *     (about 4.6 MiB).  Every GPU on which the library is loaded holds it until the process
 *     exits, whether or not this function is ever called.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, result cached per device).  Make that first call, with the device
 *     current, before starting any stream capture on that device.
 *   - All calls on a device share the one array.  Calls that can overlap on the GPU (different
 *     streams without an ordering between them, or several host threads) race on it and give
 *     wrong dw; order them on one stream or with events.  The array keeps whatever the last
 *     call left in it; this function does not depend on that content.
 *   - Return value: 0 on a successful launch, a negative code for rejected arguments
 *     (-1 shape, -2 size beyond the limit, -3 device index out of range), otherwise the CUDA
 *     error code of the failing runtime call.
 */
#ifndef CHRONICALS_B200_NOALLOC_H
#define CHRONICALS_B200_NOALLOC_H

#define CB_NOALLOC_RMSNORM_MAX_N 8192
#define CB_NOALLOC_RMSNORM_MAX_BLOCKS 148

#ifdef __cplusplus
extern "C" {
#endif

/* largest N accepted by cb_rmsnorm_bwd_noalloc */
int cb_rmsnorm_bwd_noalloc_max_n(void);

int cb_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const float* rstd, const void* dres_in,
                           void* dx, void* dw, int M, int N, float offset, int accumulate_dw, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* CHRONICALS_B200_NOALLOC_H */
