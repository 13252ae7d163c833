/* RMSNorm backward for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference framework (which has no native code at all); it
 * exists for users of this library who run inside an environment where the allocator is off limits while
 * the call is made: code running under a memory budget that was fixed at start-up, plug-ins that are handed
 * a stream by a host application and may not touch its memory pool, and replay-style loops that must not
 * trigger cudaMalloc/cudaFree (both synchronise the device).  jpb_norm_bwd() needs a caller-provided
 * scratch buffer for its per-CTA partial sums of dW; this variant keeps that scratch in a fixed array
 * inside the library image instead.
 *
 *   - Limits: H (row length) <= JPB_NOALLOC_MAX_H, H a multiple of 4 (fp32) / 8 (bf16); any number of rows.
 *     Larger H is rejected with JPB_NOALLOC_ERR_TOO_LARGE and nothing is launched.
 *   - Cost: JPB_NOALLOC_SCRATCH_BYTES of device memory on every GPU that loads the library, until exit.
 *   - The first call on a device looks up the device address of the array (cudaGetSymbolAddress); make that
 *     first call outside of any stream capture.  Later calls only launch kernels.
 *   - All calls share the one array: two calls whose kernels may overlap on the GPU (different streams
 *     without an ordering between them) race.  Calls on one stream are safe.  Nothing in the array needs to
 *     start at zero: every partial row that is read has been written earlier in the same call.
 *   - Calls no cudaMalloc / cudaFree / allocating library routine.
 *   - Speed: the partial sums come from at most JPB_NOALLOC_MAX_PARTS (148) CTAs, one per SM, so that the array stays
 *     small; jpb_norm_bwd() with a caller-provided buffer launches twice as many and is the faster of the two.
 *   - Threads: the first call on a device stores the array's address in a per-device slot without a lock.  Two host
 *     threads that make that first call at the same time both look the address up and store the same value, which is
 *     harmless; there is nothing else shared on the host side.
 *   - A positive return value is what cudaGetLastError() reports after the launches; like every use of that call it
 *     can also surface an error that an earlier, unrelated launch left pending in the context.
 */
#ifndef JAXPP_B200_NOALLOC_H
#define JAXPP_B200_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define JPB_NOALLOC_MAX_H 8192
#define JPB_NOALLOC_MAX_PARTS 148 /* CTAs that produce partial sums: one per SM of a B200 */
#define JPB_NOALLOC_SCRATCH_BYTES (JPB_NOALLOC_MAX_PARTS * 2 * JPB_NOALLOC_MAX_H * 4) /* 9.25 MiB */

#define JPB_NOALLOC_OK 0
#define JPB_NOALLOC_ERR_TOO_LARGE (-20)   /* H > JPB_NOALLOC_MAX_H */
#define JPB_NOALLOC_ERR_BAD_SHAPE (-21)   /* rows <= 0, H <= 0 or H not a multiple of the vector width */
#define JPB_NOALLOC_ERR_BAD_DTYPE (-22)
#define JPB_NOALLOC_ERR_SETUP (-23)       /* cudaGetSymbolAddress failed */

/* dtype: 0 = float32, 1 = bfloat16 (dy, x, w, dx, dw share it); rstd is float32 [rows] as returned by the
 * forward pass.  Writes dx [rows, H] and dw [H].  Returns JPB_NOALLOC_OK, one of the codes above, or a
 * positive cudaError_t from the launch. */
int jpb_rmsnorm_bwd_noalloc(int dtype, const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                            void* dw, int rows, int H, void* stream);

/* Human-readable text for a return code of jpb_rmsnorm_bwd_noalloc. */
const char* jpb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
