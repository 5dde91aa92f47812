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
/* Ping-pong between two ranks; out3[0] = nanoseconds for `iters` round trips, out3[1] = waits that gave up
 * (each wait is bounded by timeout_ms), out3[2] unused checksum.  The rank with starts = 1 sends first.
 * method 0: the sequence number is the data (st.volatile into the peer, ld.volatile of the own slot);
 * method 1: 16-byte payload + st.release.sys flag, polled with ld.acquire.sys;
 * method 2: pull, each side writes its own slot and polls the peer's.  Slots need 48 bytes. */
int fp4ar_micro_latency(void* my_slot, void* peer_slot, int iters, int starts, int method, int timeout_ms,
                        unsigned long long* out3, fp4ar_stream stream);
/* Tiles of tile_bytes written into `remote` with st.v4 and published per tile: mode 0 not at all, 1 fence.acq_rel.sys +
 * relaxed flag store, 2 st.release.sys flag store.  remote_flags: `ctas` 4-byte words in the peer's memory. */
int fp4ar_micro_publish(void* remote, void* remote_flags, size_t total_bytes, int tile_bytes, int mode, int ctas,
                        fp4ar_stream stream);
/* One thread: iters x (16-byte store into the peer [+ fence.acq_rel.sys]); out1[0] = nanoseconds. */
int fp4ar_micro_fence_cost(void* remote, int iters, int with_fence, unsigned long long* out1, fp4ar_stream stream);
/* 16-byte atomicity study.  Writer: every slot of the peer rewritten `passes` times with {i,i,i,i} (how 0: one 16-byte
 * store; 1: two 8-byte stores).  Reader: `polls` loads of every own slot (how 0: one 16-byte load; 1: two 8-byte loads);
 * out2[0] = loads whose words differ, out2[1] = value changes seen.  Neither side waits for the other. */
int fp4ar_micro_tear_writer(void* remote_slots, int nslots, int passes, int how, fp4ar_stream stream);
int fp4ar_micro_tear_reader(const void* slots, int nslots, int polls, int how, unsigned long long* out2, fp4ar_stream stream);
/* cudaMemcpyAsync device-to-device (the copy engine) between a local and a peer buffer. */
int fp4ar_micro_copy_engine(void* dst, const void* src, size_t bytes, fp4ar_stream stream);
#ifdef __cplusplus
}
#endif
#endif
