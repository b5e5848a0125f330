/* RMSNorm backward for callers that are not allowed to allocate device memory.
 *
 * This entry point has no counterpart in the reference project; it exists for embedders of this library.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a plugin inside a host application that owns
 * and budgets all device memory up front, a real-time or latency-critical loop in which an allocator call (and
 * the device synchronisation it may imply) is forbidden, or a process running under a fixed memory reservation.
 * The regular entry point, b200_rmsnorm_bwd, needs a caller-provided scratch matrix of per-CTA weight-gradient
 * partials; such callers often have no way to obtain one.  Here the scratch lives in a fixed array inside the
 * library image instead.
 *
 * Contract
 *   - computes dx = d(rmsnorm)/dx and, if dw != NULL, dw[E] = sum over rows of dy * normalised(x), exactly like
 *     b200_rmsnorm_bwd; the caller passes every input and output buffer (bf16 dy, x, dx; fp32 w, rstd, dw).
 *   - allocates nothing: no cudaMalloc / cudaFree and no allocating library routine is called, ever.
 *   - limits: E must be a multiple of 8 and at most B200_NOALLOC_MAX_E (8192); M >= 1.  dy, x, rstd and dx must
 *     not be NULL; dy, x and dx must be 16-byte aligned (rows are moved 8 bf16 values at a time; with E a
 *     multiple of 8 every row of a 16-byte aligned matrix is), w, rstd and dw 4-byte aligned.  Anything else
 *     is refused on the host, before any launch, with a negative return code and a message retrievable with
 *     b200_noalloc_last_error(); the pointers must still be device pointers of the current device.
 *   - cost: every GPU whose context loads this library holds the scratch array
 *     (B200_NOALLOC_MAX_CTAS x B200_NOALLOC_MAX_E floats = 4.6 MiB) until the process exits.
 *   - the first call on each device looks up the device address of the array (cudaGetSymbolAddress) with that
 *     device current; make this first call before starting any stream capture.
 *   - all calls on a device share the one array, which keeps the previous call's contents.  Every element that
 *     a call reads it has written itself first, so nothing needs clearing; but two calls that overlap on the
 *     GPU (different streams, or graphs replayed concurrently) race on it.  Serialise them.
 *
 * Returns 0 on success, a negative code otherwise (-1 bad size, -2 launch failure, -3 set-up failure).
 */
#ifndef B200_NOALLOC_H
#define B200_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define B200_NOALLOC_MAX_E 8192
#define B200_NOALLOC_MAX_CTAS 148

int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, void* dx, float* dw,
                             int M, int E, void* stream);

/* Human-readable reason for the last negative return code of the calling thread's most recent call. */
const char* b200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
