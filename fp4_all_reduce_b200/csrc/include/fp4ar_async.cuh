// Thin wrappers over the sm_90+/sm_100 asynchronous-copy PTX used by every kernel here:
// mbarriers, 1-D bulk copies (TMA without a tensor map), bulk-group bookkeeping, the async-proxy
// fence, programmatic dependent launch, volatile polling loads, and the error slot that every
// bounded wait reports to.  No wait in this library spins without a limit: when a limit runs out
// the waiter records where it gave up, raises a CTA-wide abort flag so later waits return at once,
// and the kernel runs to completion with a non-zero status for the host to read.
//
// The reference project has the same kind of helpers in include/codec_fast.cuh:199-226, with
// unbounded waits (kernels/push/tp2_l2.cu:330,346-363).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace fp4ar {

// ---- status words written by the device (one block of 8 words per context) ----
enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusPeerTimeout = 1,     // a receive slot still held sentinels when the wait limit ran out
  kStatusLoadTimeout = 2,     // a local bulk load did not complete in time
  kStatusBadArgument = 3,     // the kernel found inconsistent launch parameters
};
struct StatusWords {
  uint32_t code;      // first error wins (atomicCAS from 0)
  uint32_t row;       // row being waited for
  uint32_t source;    // rank whose data was missing
  uint32_t detail;    // phase: 1 one-shot gather, 2 owner reduce, 3 broadcast gather, 4 local load
  uint32_t cta;
  uint32_t call;
  uint32_t count;     // number of waits that gave up (all CTAs)
  uint32_t pad;
};

struct WaitCtx {
  StatusWords* status;            // global memory
  volatile uint32_t* cta_abort;   // shared memory flag of this CTA
  uint32_t* host_poison;          // device-mapped host word the launch path reads without a sync (may be null)
  unsigned long long limit_ns;    // how long one wait may last
  uint32_t cta, call;
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

static __device__ __noinline__ void report_wait_failure(const WaitCtx& w, uint32_t code, uint32_t row, uint32_t source,
                                                 uint32_t detail) {
  *w.cta_abort = 1u;
  if (atomicCAS(&w.status->code, 0u, code) == 0u) {
    w.status->row = row; w.status->source = source; w.status->detail = detail;
    w.status->cta = w.cta; w.status->call = w.call;
  }
  atomicAdd(&w.status->count, 1u);
  if (w.host_poison) {
    *reinterpret_cast<volatile uint32_t*>(w.host_poison) = code;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{ .reg .pred p;\n"
               "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
               "  selp.u32 %0, 1, 0, p; }"
               : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Wait for a local bulk load.  Returns false (after reporting) when the limit ran out or the CTA aborted.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, const WaitCtx& w, uint32_t row) {
  if (mbar_test(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t n = 0;
  while (!mbar_test(bar, parity)) {
    if ((++n & 63u) == 0u) {
      if (*w.cta_abort) return false;
      if (global_timer_ns() - t0 > w.limit_ns) { report_wait_failure(w, kStatusLoadTimeout, row, 0, 4); return false; }
    }
  }
  return true;
}

// ---- 1-D bulk copies (16-byte aligned addresses, sizes a multiple of 16) ----
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_addr(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Source buffers of all but the newest N groups may be overwritten.
template <int N>
__device__ __forceinline__ void bulk_wait_source_free() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// All but the newest N groups have been written to memory.
template <int N>
__device__ __forceinline__ void bulk_wait_done() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Make generic-proxy writes to shared memory visible to the async proxy (needed before a bulk store reads them).
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- programmatic dependent launch ----
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- polling loads: always served from L2 / memory, never from a stale L1 line ----
__device__ __forceinline__ uint4 poll_ld16(const void* p) {
  uint4 r;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t poll_ld2(const void* p) {
  uint16_t r;
  asm volatile("ld.volatile.global.u16 %0, [%1];" : "=h"(r) : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t poll_ld4(const void* p) {
  uint32_t r;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

__device__ __forceinline__ uint4 lds16(const void* p) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(smem_addr(p)));
  return r;
}
__device__ __forceinline__ void sts16(void* p, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(smem_addr(p)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace fp4ar
