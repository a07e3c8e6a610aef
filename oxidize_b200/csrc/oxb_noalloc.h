/* Allocation-free GEMM entry point of liboxb.
 *
 * This entry point has no counterpart in the reference project; it exists for hosts of this
 * library that must not allocate device memory themselves while they call into it: a serving
 * process whose memory pool already owns the whole GPU (every further cudaMalloc would fail or
 * fragment it), code running under a "no allocation after start-up" policy, and plain C callers
 * that have no allocator for scratch at all.  The ordinary entry point, oxb_gemm_bf16, needs the
 * caller to supply split-K scratch (fp32 partials and rendezvous counters); this one keeps that
 * scratch inside the library instead, in a fixed device array, so the caller passes only its
 * inputs and outputs.
 *
 *   Y[T, ldY >= N] (bf16) = X[T, K] (bf16, contiguous) * W[N, K]^T (bf16, contiguous) (+ bias f32[N])
 *
 * Limits and rules
 *   - T <= OXB_NOALLOC_MAX_TOKENS (one token tile).  Larger T is rejected: the call returns
 *     OXB_NOALLOC_E_TOO_LARGE and prints one line to stderr; nothing is launched.
 *   - The scratch array is OXB_NOALLOC_SCRATCH_BYTES (8 MiB + 16 KiB).  Every GPU that loads the
 *     library holds it until the process exits.  If the preferred split-K plan needs more partial
 *     space than that, fewer splits are used (same result up to fp32 summation order).
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  Make that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents.  The rendezvous
 *     counters are zeroed on the stream at the start of every call; the partials need no clearing
 *     because each is written before it is read.  Two calls that overlap on the GPU (different
 *     streams, or the same device from two threads) race on the array: serialise them.
 *   - No cudaMalloc, cudaFree or allocating library routine is called.
 *   - Any device of the process may be used (the address of the array, the SM count and the kernel's
 *     shared-memory attribute are all kept per device ordinal); each device's first call does its set-up.
 *
 * Returns 0 when the kernel was LAUNCHED, a positive cudaError_t value if a CUDA call failed, or a
 * negative OXB_NOALLOC_E_* code.  A zero return does not say that the kernel completed its work: the
 * split-K CTAs of a tile wait for one another with a bounded wait, and if other work on the GPU keeps
 * them from being resident together the wait gives up, Y is left unwritten for that tile and the
 * library's device status word records OXB_TIMEOUT_SPLITK.  Read it with oxb_status() (declared
 * below; it synchronises the device) after the call when the result matters.
 */
#ifndef OXB_NOALLOC_H
#define OXB_NOALLOC_H

#include <stddef.h>

#define OXB_NOALLOC_MAX_TOKENS 256
#define OXB_NOALLOC_COUNTER_BYTES (16 * 1024)
#define OXB_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024 + OXB_NOALLOC_COUNTER_BYTES)
#define OXB_NOALLOC_E_TOO_LARGE (-1)
#define OXB_NOALLOC_E_BAD_ARGUMENT (-2)

#ifdef __cplusplus
extern "C" {
#endif

int oxb_gemm_bf16_noalloc(const void* X, const void* W, void* Y, const float* bias, int T, int N, int K, int ldY,
                          void* cuda_stream);

/* Device status word of the library: out4 = {code, detail, count, 0}; code 0 = every bounded wait succeeded.
 * reset != 0 clears it.  Synchronises the device. */
int oxb_status(int* out4, int reset);

#ifdef __cplusplus
}
#endif
#endif /* OXB_NOALLOC_H */
