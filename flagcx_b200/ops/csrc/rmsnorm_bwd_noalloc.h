/*
 * rmsnorm_bwd_noalloc.h -- RMSNorm backward for callers that must not allocate.
 *
 * This entry point has no counterpart in the FlagCX project; it exists for users
 * of this library who run where device allocation is off the table: a serving or
 * training loop whose memory budget was fixed at start-up (every byte is planned,
 * an extra cudaMalloc can fail or fragment the pool), a latency-critical section
 * where the implicit device synchronisation of cudaMalloc/cudaFree is not
 * acceptable, or a plug-in that was handed tensors but no allocator (no torch, no
 * pool, only raw pointers and a stream).  The regular path (flagcx_b200.ops.rmsnorm backward) allocates a
 * [CTAs x hidden] fp32 scratch tensor for the per-CTA partial sums of the weight
 * gradient and a temporary for their reduction on every call; this variant keeps
 * that scratch in a fixed array inside the library instead.
 *
 *   g, x, dx : [rows, hidden] bf16, contiguous, 16-byte aligned
 *   w, dw    : [hidden] bf16
 *   rstd     : [rows] fp32 (saved by the forward)
 *
 * Limits: hidden must be a multiple of 8 and at most
 * FLAGCX_NOALLOC_RMSNORM_MAX_HIDDEN; larger sizes are refused with
 * cudaErrorInvalidValue and a message on stderr.  The scratch array is
 * FLAGCX_NOALLOC_RMSNORM_MAX_CTAS x FLAGCX_NOALLOC_RMSNORM_MAX_HIDDEN floats (4 MiB)
 * of device memory that every GPU which loads this library's device code holds until
 * the process exits.  With CUDA's default lazy module loading the array comes into
 * being when the module is first used on a device, which is the first call of this
 * entry point there: that one call may therefore make the driver set the 4 MiB aside,
 * every later call touches no allocator at all.  So make one warm-up call per device
 * at start-up, before the memory budget is fixed.
 *
 * The first call on each device also looks up the device address of that array (one
 * cudaGetSymbolAddress) and keeps it for the life of the process; after
 * cudaDeviceReset() on that device the kept address is stale and the entry point must
 * not be used again in the process.  Make the first call outside any stream capture.
 * A non-NULL stream must belong to the current device.  All calls on a device share the one array, and it keeps whatever the
 * previous call left in it: a call overwrites every slot it later reads, so
 * nothing needs clearing, but two calls that overlap on the GPU (different
 * streams without an ordering between them) race on it.  Calls on one stream are
 * safe.
 *
 * Returns cudaSuccess (0) or a cudaError_t value.  Calls no cudaMalloc, cudaFree or
 * any allocating library routine.
 */
#ifndef FLAGCX_RMSNORM_BWD_NOALLOC_H_
#define FLAGCX_RMSNORM_BWD_NOALLOC_H_

#include <stddef.h>

#define FLAGCX_NOALLOC_RMSNORM_MAX_HIDDEN 8192
#define FLAGCX_NOALLOC_RMSNORM_MAX_CTAS 128

#ifdef __cplusplus
extern "C" {
#endif

/* stream: a cudaStream_t (NULL for the default stream). */
int flagcxRmsnormBwdNoAlloc(const void *g, const void *x, const void *w, const float *rstd, void *dx, void *dw,
                            long rows, int hidden, void *stream);

#ifdef __cplusplus
}
#endif
#endif
