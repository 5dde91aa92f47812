/* fp4ar_reduce_reencode_noalloc: the two-shot owner step for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference project.
 *
 * Who needs it: code that runs where device memory cannot be requested -- a plugin invoked inside another
 * framework's memory plan, a callback running under a captured or otherwise frozen allocator state, a
 * real-time loop that forbids anything that may take the driver's allocation lock.  fp4ar_reduce_reencode()
 * wants a [rows][3584] record buffer from its caller even when the caller only needs the BF16 result; here
 * that buffer is a fixed array inside the library.
 *
 * What it does: out[r] = decode(encode(sum over sources of decode(source[r]))) for rows r < rows, the same
 * values, bit for bit, as the `out_bf16` of fp4ar_reduce_reencode().  The re-encoded records stay in the
 * library's array and are not returned.
 *
 * Limits and rules
 *  - rows <= FP4AR_NOALLOC_MAX_ROWS; larger calls return FP4AR_ERR_ARGUMENT and launch nothing.
 *    fp4ar_noalloc_last_error() then holds a sentence saying so.
 *  - The array (FP4AR_NOALLOC_MAX_ROWS x 3584 bytes, about 3.5 MiB) is resident on every GPU that loads the
 *    library, until the process exits.
 *  - The function calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on a
 *    device looks up the array's device address (cudaGetSymbolAddress); make that first call with the device
 *    current and before any stream capture begins.  Later calls on that device take no lock and make no CUDA
 *    call other than cudaGetDevice, the launch and cudaGetLastError.  The address is remembered per device for
 *    the life of the process: after cudaDeviceReset() on a device it is stale, and this entry point must not
 *    be used on that device again.
 *  - Every call on a device shares the one array, which keeps the previous call's records.  Nothing in it has
 *    to start at zero (each call overwrites every byte it later reads), but two calls that overlap on the
 *    GPU -- different streams, or different host threads -- race on it: serialise them.
 */
#ifndef FP4AR_NOALLOC_H_
#define FP4AR_NOALLOC_H_

#include "fp4ar.h"

#ifdef __cplusplus
extern "C" {
#endif

#define FP4AR_NOALLOC_MAX_ROWS 1024

/* Arguments as fp4ar_reduce_reencode() without rec_out.  Returns FP4AR_OK or an FP4AR_ERR_* code. */
int fp4ar_reduce_reencode_noalloc(int nsrc, const void* const* src, long pitch, const float* const* rs,
                                  const float* gs, int rows, void* out_bf16, fp4ar_stream stream);

/* Text of the last error this entry point reported on the calling thread ("" if none). */
const char* fp4ar_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* FP4AR_NOALLOC_H_ */
