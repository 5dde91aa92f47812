/* Row-parallel GEMM with an NVFP4 epilogue feeding the AllReduce windows (B200, tcgen05 / TMEM).
 *
 *   partial = X[M,K] x Wt[N,K]^T   (BF16 in, FP32 accumulate), quantised per 16 outputs with the static scale gs
 *
 * push != NULL : the row pieces are stored into the receive windows described by the push view of an
 *                AllReduce context (fp4ar_get_push_view): every rank's window for the one-shot algorithm,
 *                the row owner's window (row % nranks) for the two-shot algorithm.  Follow it on the same
 *                stream with fp4ar_launch(..., input = FP4AR_IN_PUSHED, gs = {all ranks' scales}).  N must be 6144.
 * local_q      : optional [M][N/2 + N/16] NVFP4 rows (values then scales) written locally.
 * dbg_acc      : optional [M][N] FP32 dump of the accumulators (for verification).
 * Requirements : K multiple of 64, N multiple of 256, X and Wt 16-byte aligned and K-contiguous.
 *
 * The reference project has no producer of this kind (README.md:76); its harness emulates one with a copy.
 */
#ifndef FP4AR_GEMM_H_
#define FP4AR_GEMM_H_

#include "fp4ar.h"

#ifdef __cplusplus
extern "C" {
#endif

int fp4ar_gemm_nvfp4(const fp4ar_push_view* push, int two_shot, const void* x, const void* wt, int M, int N, int K,
                     float gs, void* local_q, float* dbg_acc, fp4ar_stream stream);
/* Status block of the GEMM kernels on the current device (code != 0: a bounded wait gave up). */
int fp4ar_gemm_status(fp4ar_status_words* out);
/* After a GEMM whose status is not 0: waits for the device, then clears the status block and the hand-off flags of the
 * partial tiles that such a launch may have left set (a later launch would wait on them until its limit). */
int fp4ar_gemm_reset(void);
/* The schedule a call of this size takes on a device with `sms` SMs (host only, no device work; environment overrides
 * are not applied): CTA pairs or single CTAs, tile width, whether the K loop is cut across units (stream-K), how many
 * units (CTAs or pairs) work on how many tiles.  With `segments` != NULL also the work list of unit `unit` as
 * quadruples (tile, first K block, K blocks, kind: 0 whole tile, 1 leaves a partial, 2 adds the next unit's partial);
 * returns the number of segments (also when it exceeds max_segments), 0 without a list, -1 for bad arguments. */
int fp4ar_gemm_plan(int M, int N, int K, int sms, int* pair, int* tile_n, int* stream_k, int* units, int* tiles,
                    int unit, int* segments, int max_segments);

#ifdef __cplusplus
}
#endif
#endif /* FP4AR_GEMM_H_ */
