// NVLink transport micro-benchmarks: what a kernel can push into (or pull from) a peer's memory, and how long
// one hand-off takes.  They fix the "payload ceiling" that the fused kernels are measured against.
//
//   bandwidth  method 0  bulk asynchronous store shared -> peer global (cp.async.bulk, the fused kernels' egress)
//              method 1  st.global.v4 from registers
//              method 2  bulk asynchronous load peer global -> shared (a pull; plain, per-CTA)
//              method 3  multimem.st.v4.f32 to a multicast mapping (in-switch broadcast to every rank)
//   latency    ping-pong of a sequence number through one 16-byte slot per direction, receiver polling with
//              volatile loads (the Lamport style hand-off), bounded waits; variants: payload + st.release.sys flag
//              polled with ld.acquire.sys, and a pull (each side polls the PEER's memory)
//   fence      cost of publishing tiles written into a peer: nothing / fence.acq_rel.sys + flag / st.release.sys flag
//              per tile, and nanoseconds per (remote store + fence.acq_rel.sys) from one thread
//   tear       do 16-byte stores into a peer arrive whole?  A writer rewrites slots with {i,i,i,i}; the reader counts
//              16-byte loads whose four words differ (and, as the control, pairs of 8-byte loads)
//
// Counterparts in the reference project: bench/micro/bw.cu:16-90, bench/micro/lat.cu:16-64,
// bench/micro/fence.cu:31-82, bench/micro/tear.cu:17-97, bench/link/ce.cu:15-22 (SM copy versus copy engine).
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

// One thread per rank.  The rank with starts = 1 sends first; each side waits for sequence i, then answers with i.
//   method 0  Lamport style: the sequence number IS the data, written with st.volatile into the peer's slot,
//             the receiver polls its own memory with ld.volatile
//   method 1  flag style: 16-byte payload into the peer, then st.release.sys of a flag; the receiver polls the flag
//             with ld.acquire.sys and reads the payload afterwards
//   method 2  pull: each side writes its OWN slot and polls the peer's slot across the link
// out[0] = total nanoseconds on this rank, out[1] = number of waits that gave up.
__global__ void micro_latency_kernel(uint32_t* my_slot, uint32_t* peer_slot, int iters, int starts, int method,
                                     unsigned long long limit_ns, unsigned long long* out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  unsigned long long gave_up = 0;
  uint32_t sink = 0;
  const unsigned long long t0 = global_timer_ns();
  auto send = [&](uint32_t i) {
    if (method == 0) {
      asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(peer_slot), "r"(i) : "memory");
    } else if (method == 1) {
      asm volatile("st.global.v4.u32 [%0], {%1, %1, %1, %1};" ::"l"(peer_slot + 8), "r"(i) : "memory");
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_slot), "r"(i) : "memory");
    } else {
      asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(my_slot), "r"(i) : "memory");
    }
  };
  auto seen = [&](uint32_t i) -> bool {
    uint32_t v;
    if (method == 0) {
      asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(my_slot) : "memory");
    } else if (method == 1) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_slot) : "memory");
      if (v == i) { uint32_t d; asm volatile("ld.global.u32 %0, [%1];" : "=r"(d) : "l"(my_slot + 8) : "memory"); sink += d; }
    } else {
      asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(peer_slot) : "memory");
    }
    return v == i;
  };
  for (int i = 1; i <= iters; i++) {
    if (starts) send((uint32_t)i);
    const unsigned long long w0 = global_timer_ns();
    uint32_t n = 0;
    while (!seen((uint32_t)i)) {
      if ((++n & 255u) == 0u && global_timer_ns() - w0 > limit_ns) { gave_up++; break; }
    }
    if (gave_up) break;
    if (!starts) send((uint32_t)i);
  }
  out[0] = global_timer_ns() - t0;
  out[1] = gave_up;
  out[2] = sink;
}

// Publication cost.  Every CTA writes its tiles of `tile_bytes` into the peer with st.v4 and publishes each tile:
//   mode 0 nothing; 1 __syncthreads + fence.acq_rel.sys + st.relaxed flag (thread 0); 2 __syncthreads +
//   st.release.sys flag (thread 0).  flags: one 4-byte word per CTA in the peer's memory.
__global__ void __launch_bounds__(kMicroThreads, 1)
micro_publish_kernel(char* remote, uint32_t* remote_flags, size_t total, int tile_bytes, int mode) {
  const uint4 v = make_uint4(0x11111111u, 0x22222222u, 0x33333333u, 0x44444444u);
  const size_t ntiles = total / tile_bytes;
  uint32_t seq = 0;
  for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    uint4* d = reinterpret_cast<uint4*>(remote + t * tile_bytes);
    for (int i = threadIdx.x; i < tile_bytes / 16; i += blockDim.x) d[i] = v;
    if (mode != 0) {
      __syncthreads();
      if (threadIdx.x == 0) {
        seq++;
        if (mode == 1) {
          asm volatile("fence.acq_rel.sys;" ::: "memory");
          asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(remote_flags + blockIdx.x), "r"(seq) : "memory");
        } else {
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote_flags + blockIdx.x), "r"(seq) : "memory");
        }
      }
    }
  }
}

// One thread: `iters` times (16-byte store into the peer, then fence.acq_rel.sys when with_fence).  out[0] = ns.
__global__ void micro_fence_cost_kernel(char* remote, int iters, int with_fence, unsigned long long* out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const unsigned long long t0 = global_timer_ns();
  for (int i = 0; i < iters; i++) {
    asm volatile("st.global.v4.u32 [%0], {%1, %1, %1, %1};" ::"l"(remote + 16 * (i & 1023)), "r"((uint32_t)i) : "memory");
    if (with_fence) asm volatile("fence.acq_rel.sys;" ::: "memory");
  }
  out[0] = global_timer_ns() - t0;
}

// Tear study, writer side: `passes` times, every thread rewrites its slot in the peer with {i,i,i,i}.
//   how 0: one st.global.v4 (16 bytes)    how 1: two st.global.v2 (8 + 8 bytes; may legitimately tear)
__global__ void micro_tear_writer_kernel(uint4* remote_slots, int nslots, int passes, int how) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= nslots) return;
  for (int i = 1; i <= passes; i++) {
    const uint32_t w = (uint32_t)i;
    if (how == 0) {
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %1, %1, %1};" ::"l"(remote_slots + s), "r"(w) : "memory");
    } else {
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %1};" ::"l"(remote_slots + s), "r"(w) : "memory");
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %1};" ::"l"(reinterpret_cast<char*>(remote_slots + s) + 8), "r"(w) : "memory");
    }
  }
}

// Tear study, reader side: `polls` loads of each slot of the OWN buffer; nothing waits on the writer.
//   how 0: one ld.volatile.v4      how 1: two ld.volatile.v2
// out[0] = loads whose four words differ, out[1] = loads that saw a value other than the previous one (progress).
__global__ void micro_tear_reader_kernel(const uint4* slots, int nslots, int polls, int how, unsigned long long* out) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= nslots) return;
  unsigned long long torn = 0, changes = 0;
  uint32_t last = 0;
  for (int i = 0; i < polls; i++) {
    uint4 v;
    if (how == 0) {
      asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(slots + s) : "memory");
    } else {
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(slots + s) : "memory");
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.z), "=r"(v.w) : "l"(reinterpret_cast<const char*>(slots + s) + 8) : "memory");
    }
    if (v.x != v.y || v.x != v.z || v.x != v.w) torn++;
    if (v.x != last) { changes++; last = v.x; }
  }
  if (torn) atomicAdd(out, torn);
  if (changes) atomicAdd(out + 1, changes);
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

extern "C" int fp4ar_micro_latency(void* my_slot, void* peer_slot, int iters, int starts, int method, int timeout_ms,
                                   unsigned long long* out3, fp4ar_stream stream) {
  if (!my_slot || !peer_slot || iters < 1 || !out3 || method < 0 || method > 2) return FP4AR_ERR_ARGUMENT;
  micro_latency_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint32_t*)my_slot, (uint32_t*)peer_slot, iters, starts, method,
                                                           (unsigned long long)timeout_ms * 1000000ull, out3);
  return cuda_check_launch();
}

extern "C" int fp4ar_micro_publish(void* remote, void* remote_flags, size_t total_bytes, int tile_bytes, int mode, int ctas,
                                   fp4ar_stream stream) {
  if (!remote || !remote_flags || tile_bytes < 16 || (tile_bytes & 15) || mode < 0 || mode > 2 || ctas < 1 || ctas > 1024 ||
      total_bytes < (size_t)tile_bytes)
    return FP4AR_ERR_ARGUMENT;
  micro_publish_kernel<<<ctas, kMicroThreads, 0, (cudaStream_t)stream>>>((char*)remote, (uint32_t*)remote_flags, total_bytes,
                                                                         tile_bytes, mode);
  return cuda_check_launch();
}

extern "C" int fp4ar_micro_fence_cost(void* remote, int iters, int with_fence, unsigned long long* out1, fp4ar_stream stream) {
  if (!remote || iters < 1 || !out1) return FP4AR_ERR_ARGUMENT;
  micro_fence_cost_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((char*)remote, iters, with_fence, out1);
  return cuda_check_launch();
}

extern "C" int fp4ar_micro_tear_writer(void* remote_slots, int nslots, int passes, int how, fp4ar_stream stream) {
  if (!remote_slots || nslots < 1 || passes < 1 || how < 0 || how > 1) return FP4AR_ERR_ARGUMENT;
  micro_tear_writer_kernel<<<(nslots + 255) / 256, 256, 0, (cudaStream_t)stream>>>((uint4*)remote_slots, nslots, passes, how);
  return cuda_check_launch();
}

extern "C" int fp4ar_micro_tear_reader(const void* slots, int nslots, int polls, int how, unsigned long long* out2,
                                       fp4ar_stream stream) {
  if (!slots || nslots < 1 || polls < 1 || how < 0 || how > 1 || !out2) return FP4AR_ERR_ARGUMENT;
  micro_tear_reader_kernel<<<(nslots + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const uint4*)slots, nslots, polls, how, out2);
  return cuda_check_launch();
}

// Copy engine: a plain asynchronous device-to-device copy issued by the runtime (no SM kernel), for comparison.
extern "C" int fp4ar_micro_copy_engine(void* dst, const void* src, size_t bytes, fp4ar_stream stream) {
  if (!dst || !src || bytes == 0) return FP4AR_ERR_ARGUMENT;
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream) != cudaSuccess) return cuda_fail();
  return FP4AR_OK;
}
