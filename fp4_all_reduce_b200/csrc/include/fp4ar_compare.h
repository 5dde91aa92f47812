/* Comparison variants of the NVFP4 AllReduce (see csrc/kernels/compare_variants.cu): a flag-based push (the
 * control), pulls with BF16 and with NVFP4 input, a two-shot by pull, and a pull reduce-scatter with a pushed
 * all-gather.  Same records and arithmetic as the main operator (bit-identical to its one-shot / two-shot host
 * model); they exist to put numbers on the hand-off designs the main kernel does not use. */
#ifndef FP4AR_COMPARE_H_
#define FP4AR_COMPARE_H_
#include "fp4ar.h"
#ifdef __cplusplus
extern "C" {
#endif
/* Bytes of the (zero-initialised, 256-byte aligned, peer-mapped) window each rank needs. */
size_t fp4ar_compare_window_bytes(int max_rows, int nranks);
/* One AllReduce of `rows` x 6144 (BF16 out).  variant 0: flag push, 1: pull, 2: pull with NVFP4 input (x = [rows][3456]
 * NVFP4 rows, gs = every rank's static scale; x is BF16 [rows][6144] and gs unused otherwise), 3: two-shot by pull,
 * 4: pull reduce-scatter + push all-gather.
 * nlocal == 1: this process is `rank`; x/out/status have one entry.  nlocal == nranks: all ranks are emulated on
 * the current device as CTA groups of one cooperative launch; x/out/status have one entry per rank and `rank` is
 * ignored.  windows: every rank's window (peer-mapped addresses, or all local when emulated).  status: device
 * memory, zero-initialised; first failed wait is recorded there.  Every rank must make the same sequence of calls
 * on windows that started zeroed (the generation counter lives in the window). */
int fp4ar_compare_allreduce(int variant, int rank, int nranks, int nlocal, void* const* windows, size_t window_bytes,
                            int max_rows, const void* const* x, void* const* out, int rows, const float* gs,
                            fp4ar_status_words* const* status, int timeout_ms, fp4ar_stream stream);
#ifdef __cplusplus
}
#endif
#endif
