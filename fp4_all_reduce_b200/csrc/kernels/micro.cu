// NVLink transport micro-benchmarks: what a kernel can push into (or pull from) a peer's memory, and how long
// one hand-off takes.  They fix the "payload ceiling" that the fused kernels are measured against.
//
//   bandwidth  method 0  bulk asynchronous store shared -> peer global (cp.async.bulk, the fused kernels' egress)
//              method 1  st.global.v4 from registers
//              method 2  bulk asynchronous load peer global -> shared (a pull; plain, per-CTA)
//              method 3  multimem.st.v4.f32 to a multicast mapping (in-switch broadcast to every rank)
//   latency    ping-pong of a sequence number through one 16-byte slot per direction, receiver polling with
//              volatile loads (the Lamport style hand-off), bounded waits
//
// Counterparts in the reference project: bench/micro/bw.cu:16-90, bench/micro/lat.cu:16-64,
// bench/link/ce.cu:15-22 (SM copy versus copy engine).
#include <cuda_runtime.h>
#include "../include/fp4ar.h"
#include "../include/fp4ar_async.cuh"
#include "../include/fp4ar_micro.h"
#include "host_util.h"

namespace fp4ar {

constexpr int kMicroThreads = 256;
constexpr int kMicroMaxChunk = 32768;

__global__ void __launch_bounds__(kMicroThreads, 1)
micro_bw_kernel(char* remote, char* local_scratch, size_t total, int chunk, int method, int inflight) {
  extern __shared__ __align__(128) uint8_t sm[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm);                 // [8] for the pull ring
  uint8_t* buf = sm + 128;
  const size_t nchunks = total / chunk;
  if (method == 0) {
    for (int i = threadIdx.x; i < chunk / 16; i += blockDim.x)
      reinterpret_cast<uint4*>(buf)[i] = make_uint4(0x11111111u, 0x22222222u, 0x33333333u, 0x44444444u);
    fence_smem_to_async();
    __syncthreads();
    if (threadIdx.x == 0) {
      int pending = 0;
      for (size_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        bulk_store(remote + c * chunk, buf, (uint32_t)chunk);
        bulk_commit();
        if (++pending >= inflight) { bulk_wait_source_free<0>(); pending = 0; }
      }
      bulk_wait_done<0>();
    }
  } else if (method == 1) {
    const uint4 v = make_uint4(0x11111111u, 0x22222222u, 0x33333333u, 0x44444444u);
    for (size_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
      uint4* d = reinterpret_cast<uint4*>(remote + c * chunk);
      for (int i = threadIdx.x; i < chunk / 16; i += blockDim.x) d[i] = v;
    }
  } else if (method == 2) {
    constexpr int kRing = 4;
    if (threadIdx.x == 0) { for (int i = 0; i < kRing; i++) mbar_init(bars + i, 1); mbar_init_fence(); }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t issued = 0, waited = 0;
      for (size_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        if (issued - waited == (uint32_t)kRing) {
          uint32_t spins = 0;
          while (!mbar_test(bars + (waited % kRing), (waited / kRing) & 1u) && ++spins < (1u << 26)) {}
          waited++;
        }
        const int s = issued % kRing;
        mbar_arrive_expect(bars + s, (uint32_t)chunk);
        bulk_load(buf + (size_t)s * chunk, remote + c * chunk, (uint32_t)chunk, bars + s);
        issued++;
      }
      while (waited < issued) {
        uint32_t spins = 0;
        while (!mbar_test(bars + (waited % kRing), (waited / kRing) & 1u) && ++spins < (1u << 26)) {}
        waited++;
      }
    }
  } else {
    for (size_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
      char* d = remote + c * chunk;
      for (int i = threadIdx.x; i < chunk / 16; i += blockDim.x)
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + 16 * (size_t)i), "f"(1.0f),
                     "f"(2.0f), "f"(3.0f), "f"(4.0f)
                     : "memory");
    }
  }
  (void)local_scratch;
}

// One thread per rank.  Rank `first` starts; each side waits for sequence i in its own slot, then writes i into the
// peer's slot.  out[0] = total nanoseconds on this rank, out[1] = number of waits that gave up.
__global__ void micro_latency_kernel(volatile uint32_t* my_slot, uint32_t* peer_slot, int iters, int starts,
                                     unsigned long long limit_ns, unsigned long long* out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  unsigned long long gave_up = 0;
  const unsigned long long t0 = global_timer_ns();
  for (int i = 1; i <= iters; i++) {
    if (starts) {
      asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(peer_slot), "r"((uint32_t)i) : "memory");
    }
    const unsigned long long w0 = global_timer_ns();
    uint32_t n = 0;
    while (*my_slot != (uint32_t)i) {
      if ((++n & 255u) == 0u && global_timer_ns() - w0 > limit_ns) { gave_up++; break; }
    }
    if (!starts) {
      asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(peer_slot), "r"((uint32_t)i) : "memory");
    }
    if (gave_up) break;
  }
  out[0] = global_timer_ns() - t0;
  out[1] = gave_up;
}

}  // namespace fp4ar

using namespace fp4ar;

extern "C" int fp4ar_micro_bandwidth(void* remote, size_t total_bytes, int chunk_bytes, int method, int ctas,
                                     int inflight, fp4ar_stream stream) {
  if (!remote || chunk_bytes < 16 || (chunk_bytes & 15) || chunk_bytes > kMicroMaxChunk || method < 0 || method > 3 ||
      ctas < 1 || total_bytes < (size_t)chunk_bytes || inflight < 1)
    return FP4AR_ERR_ARGUMENT;
  const int smem = 128 + (method == 2 ? 4 * chunk_bytes : chunk_bytes);
  if (cudaFuncSetAttribute(micro_bw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return cuda_fail();
  micro_bw_kernel<<<ctas, kMicroThreads, smem, (cudaStream_t)stream>>>((char*)remote, nullptr, total_bytes, chunk_bytes,
                                                                       method, inflight);
  return cuda_check_launch();
}

extern "C" int fp4ar_micro_latency(void* my_slot, void* peer_slot, int iters, int starts, int timeout_ms,
                                   unsigned long long* out2, fp4ar_stream stream) {
  if (!my_slot || !peer_slot || iters < 1 || !out2) return FP4AR_ERR_ARGUMENT;
  micro_latency_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((volatile uint32_t*)my_slot, (uint32_t*)peer_slot, iters, starts,
                                                           (unsigned long long)timeout_ms * 1000000ull, out2);
  return cuda_check_launch();
}
