/* NVLink transport micro-benchmarks (see csrc/kernels/micro.cu). */
#ifndef FP4AR_MICRO_H_
#define FP4AR_MICRO_H_
#include "fp4ar.h"
#ifdef __cplusplus
extern "C" {
#endif
/* method 0 bulk store, 1 st.v4, 2 bulk load (pull), 3 multimem.st (remote = multicast address).
 * Moves total_bytes in chunks of chunk_bytes (16..32768, multiple of 16) with `ctas` CTAs; `inflight` bounds the
 * bulk stores a CTA keeps outstanding. */
int fp4ar_micro_bandwidth(void* remote, size_t total_bytes, int chunk_bytes, int method, int ctas, int inflight,
                          fp4ar_stream stream);
/* Ping-pong through one 4-byte slot per direction; out2[0] = nanoseconds for `iters` round trips, out2[1] = waits
 * that gave up.  The rank with starts = 1 sends first. */
int fp4ar_micro_latency(void* my_slot, void* peer_slot, int iters, int starts, int timeout_ms, unsigned long long* out2,
                        fp4ar_stream stream);
#ifdef __cplusplus
}
#endif
#endif
