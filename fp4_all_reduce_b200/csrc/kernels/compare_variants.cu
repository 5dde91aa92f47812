// Comparison variants of the one-shot NVFP4 AllReduce, kept to measure the design choices of the main kernel
// against their classic alternatives.  Same wire records, same arithmetic (bit-identical to the one-shot host
// model), different hand-off:
//
//   variant 0  "flag push" (the control): every row is encoded and written into every rank's window with plain
//              16-byte stores; per (source, tile of 4 rows) one st.release.sys flag carries the call generation;
//              consumers spin on the flags in their own memory with ld.acquire.sys, then decode from local memory.
//   variant 1  "pull": every row is encoded into the rank's OWN window and published with a local flag; consumers
//              poll the producer's flag across the link, then pull the record into shared memory with a plain
//              (non-multicast, per-warp) bulk asynchronous load and decode from there.
//
//   variant 2  "pull, NVFP4 input": the producer's NVFP4 rows (static per-rank scale, no row scale) are copied into
//              the rank's own window slot and published like variant 1; consumers pull 3456-byte records and decode
//              them with the static scales.
//   variant 3  "two-shot pull": every rank encodes all its rows into its own window (reduce-scatter data); the owner
//              of a row (row % P) pulls the other ranks' records of that row, sums in rank order, re-encodes, writes
//              the re-encoding into its own window and publishes a per-row flag; every other rank pulls the
//              re-encoding.  Every rank, the owner too, outputs the decode of the re-encoding.
//   variant 4  "pull reduce-scatter, push all-gather": as variant 3, but the owner stores the re-encoding into every
//              peer's window and sets the per-row flag there, so the consumers poll and read local memory.
//
// Against the main kernel: no sentinels and no re-arm, but a system-scope release per tile, a generation counter,
// a second round trip before any byte is consumed (pull), and no overlap between the encode of a tile and the
// waits of the previous one.  One warp per row, 4 rows per CTA step.
//
// Call state: window-resident generation counter `gen` (calls completed by this rank).  Buffer = gen & 1, flag
// value = gen + 1.  Two buffers are enough: a rank reaches call n + 2 only after its call n + 1 saw every peer's
// flags of call n + 1, and a peer publishes those only after its own call n has ended.  The last CTA of a rank to
// finish advances `gen` (a ticket in the same control block), so a captured graph replays without host state.
//
// Every wait is bounded by `timeout_ns`; a wait that gives up records {code, row, source, detail} in the status
// block and the row is skipped.
//
// Reference project counterparts: kernels/control/r1.cu:139-176 (flag control, one-shot), :130-137 (generation
// counter at grid exit); kernels/pull/tp2_p.cu:211-614 (pull); kernels/pull/tp2_pq.cu:66-212 and tp4_p4q.cu:67-210
// (pull with NVFP4 input); kernels/pull/tp4_p4.cu:225-704 (two-shot pull) and :620-656 (all-gather by push).
#include <cuda_runtime.h>
#include <cstring>
#include "../include/fp4ar.h"
#include "../include/fp4ar_compare.h"
#include "host_util.h"
#include "row_ops.cuh"

namespace fp4ar {

constexpr int kCmpWarps = 4;                       // rows per CTA step
constexpr int kCmpWarpBytes = 4 * kRowB + 64;      // x row, 2 x 12 KB record area (8 x 3584 B), output staging
constexpr int kCmpSmem = kCmpWarps * kCmpWarpBytes + 16;

struct CmpRank {
  const char* x;
  char* out;
  StatusWords* status;
  int rank;
};
struct CmpParams {
  CmpRank io[kMaxRanksOps];        // one per LOCAL rank (1, or P when the ranks are emulated on one GPU)
  char* win[kMaxRanksOps];         // every rank's window
  int rows, cap, ntiles_cap, ctas_per_rank, nranks;
  unsigned long long timeout_ns;
  float gs[kMaxRanksOps];          // NVFP4 input: static scale of every rank's rows
};

// window layout: [2][P][cap] records | [2][P][ntiles_cap] tile flags | control {gen, ticket} | [2][cap] row flags
__host__ __device__ inline size_t cmp_flags_offset(int P, int cap) { return (size_t)2 * P * cap * kRecStride; }
__host__ __device__ inline size_t cmp_ctrl_offset(int P, int cap, int ntiles_cap) {
  return cmp_flags_offset(P, cap) + (((size_t)2 * P * ntiles_cap * 4 + 255) & ~(size_t)255);
}

__host__ __device__ inline size_t cmp_rowflag_offset(int P, int cap, int ntiles_cap) {
  return cmp_ctrl_offset(P, cap, ntiles_cap) + 256;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int P, int PULL, int QIN>
__global__ void __launch_bounds__(kCmpWarps * 32, 1) cmp_kernel(const __grid_constant__ CmpParams prm) {
  static_assert(!QIN || PULL, "NVFP4 input is built for the pull variant");
  constexpr uint32_t kPullBytes = QIN ? kQRowBytes : kRecPayload;
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int f = (lane >> 1) & 3;
  const int local = blockIdx.x / prm.ctas_per_rank, cta = blockIdx.x - local * prm.ctas_per_rank;
  const CmpRank io = prm.io[local];
  const int me = io.rank;
  uint8_t* base = smem + (size_t)warp * kCmpWarpBytes;
  uint8_t* xbuf = base;                          // 12 KB
  uint8_t* recs = base + kRowB;                  // 24 KB: up to 6 records; with 8 ranks the x buffer is reused too
  uint8_t* obuf = base + 3 * kRowB;              // 12 KB
  uint64_t* bar = reinterpret_cast<uint64_t*>(base + 4 * kRowB);   // [0] x row, [1] pulled records
  uint32_t* err_word = reinterpret_cast<uint32_t*>(smem + (size_t)kCmpWarps * kCmpWarpBytes);
  if (lane == 0) { mbar_init(bar, 1); mbar_init(bar + 1, 1); }
  if (threadIdx.x == 0) *err_word = 0u;
  mbar_init_fence();
  __syncthreads();

  char* my_win = prm.win[me];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(my_win + cmp_ctrl_offset(P, prm.cap, prm.ntiles_cap));
  const uint32_t gen = *reinterpret_cast<volatile uint32_t*>(ctrl);
  const uint32_t want = gen + 1u;
  const size_t buf_rec = (size_t)(gen & 1u) * P * prm.cap * kRecStride;
  const size_t buf_flag = cmp_flags_offset(P, prm.cap) + (size_t)(gen & 1u) * P * prm.ntiles_cap * 4;
  const int ntiles = (prm.rows + kCmpWarps - 1) / kCmpWarps;

  uint32_t xphase = 0, rphase = 0;
  bool pending_store = false;
  for (int t = cta; t < ntiles; t += prm.ctas_per_rank) {
    const int row = t * kCmpWarps + warp;
    const bool live = row < prm.rows;
    // ---------------------------------------------------------------- produce
    if (live && QIN) {
      // the producer's NVFP4 row (3456 B) goes into this rank's own window record as it is
      const size_t rec_off = buf_rec + ((size_t)me * prm.cap + row) * kRecStride;
      const char* src = io.x + (size_t)row * kQRowBytes;
      for (int c = lane; c < kQRowBytes / 16; c += 32)
        *reinterpret_cast<uint4*>(my_win + rec_off + 16 * c) = __ldg(reinterpret_cast<const uint4*>(src + 16 * c));
    }
    if (live && !QIN) {
      if (lane == 0) { mbar_arrive_expect(bar, kRowB); bulk_load(xbuf, io.x + (size_t)row * kRowB, kRowB, bar); }
      wait_row(bar, xphase & 1u, err_word);
      xphase++;
      const size_t rec_off = buf_rec + ((size_t)me * prm.cap + row) * kRecStride;
      float rs;
      encode_row_from_smem(xbuf, lane, 0.0f, false, rs,
                           [&](int p, uint4 q) {
                             if (PULL) { *reinterpret_cast<uint4*>(my_win + rec_off + 16 * p) = q; }
                             else {
#pragma unroll
                               for (int d = 0; d < P; d++) *reinterpret_cast<uint4*>(prm.win[d] + rec_off + 16 * p) = q;
                             }
                           },
                           [&](int p, uint32_t sf2) {
                             if (PULL) { *reinterpret_cast<uint16_t*>(my_win + rec_off + kValueBytes + 2 * p) = (uint16_t)sf2; }
                             else {
#pragma unroll
                               for (int d = 0; d < P; d++)
                                 *reinterpret_cast<uint16_t*>(prm.win[d] + rec_off + kValueBytes + 2 * p) = (uint16_t)sf2;
                             }
                           });
      if (lane == 0) {
        const uint32_t b = __float_as_uint(rs);
        const uint4 r4 = make_uint4(b, b, b, b);
        if (PULL) { *reinterpret_cast<uint4*>(my_win + rec_off + kQRowBytes) = r4; }
        else {
#pragma unroll
          for (int d = 0; d < P; d++) *reinterpret_cast<uint4*>(prm.win[d] + rec_off + kQRowBytes) = r4;
        }
      }
    }
    __syncthreads();                               // the tile's stores happen-before the release below
    if (PULL) {
      if (threadIdx.x == 0) st_release_sys(reinterpret_cast<uint32_t*>(my_win + buf_flag) + (size_t)me * prm.ntiles_cap + t, want);
    } else {
      if (threadIdx.x < P)
        st_release_sys(reinterpret_cast<uint32_t*>(prm.win[threadIdx.x] + buf_flag) + (size_t)me * prm.ntiles_cap + t, want);
    }
    // ---------------------------------------------------------------- consume
    if (live) {
      bool ok = true;
      // flags of every source for this tile: in the own window (push) or in the producer's (pull)
#pragma unroll 1
      for (int s = 0; s < P && ok; s++) {
        const uint32_t* fl = reinterpret_cast<const uint32_t*>((PULL ? prm.win[s] : my_win) + buf_flag) + (size_t)s * prm.ntiles_cap + t;
        if (ld_acquire_sys(fl) != want) {
          const unsigned long long t0 = global_timer_ns();
          uint32_t n = 0;
          while (ld_acquire_sys(fl) != want) {
            if ((++n & 63u) == 0u && global_timer_ns() - t0 > prm.timeout_ns) {
              if (lane == 0) {
                if (atomicCAS(&io.status->code, 0u, (uint32_t)kStatusPeerTimeout) == 0u) {
                  io.status->row = (uint32_t)row; io.status->source = (uint32_t)s; io.status->detail = 1u;
                  io.status->cta = (uint32_t)cta; io.status->call = gen;
                }
                atomicAdd(&io.status->count, 1u);
              }
              ok = false;
              break;
            }
          }
        }
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        const char* src_base[P];
        if (PULL) {
          // pull every source's record into shared memory (the x buffer is free again: 36 KB hold 8 records)
          __syncwarp();
          if (lane == 0) {
            // the records were written through the generic proxy (by another GPU) and are read by the async proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
            mbar_arrive_expect(bar + 1, (uint32_t)P * kPullBytes);
#pragma unroll
            for (int s = 0; s < P; s++) {
              uint8_t* dst = (s < 6 ? recs + s * kRecStride : xbuf + (s - 6) * kRecStride);
              bulk_load(dst, prm.win[s] + buf_rec + ((size_t)s * prm.cap + row) * kRecStride, kPullBytes, bar + 1);
            }
          }
          wait_row(bar + 1, rphase & 1u, err_word);
          rphase++;
#pragma unroll
          for (int s = 0; s < P; s++) src_base[s] = reinterpret_cast<const char*>(s < 6 ? recs + s * kRecStride : xbuf + (s - 6) * kRecStride);
        } else {
#pragma unroll
          for (int s = 0; s < P; s++) src_base[s] = my_win + buf_rec + ((size_t)s * prm.cap + row) * kRecStride;
        }
        float rsv[P];
#pragma unroll
        for (int s = 0; s < P; s++)
          rsv[s] = QIN ? prm.gs[s]
                       : (PULL ? *reinterpret_cast<const float*>(src_base[s] + kQRowBytes)
                               : __ldcg(reinterpret_cast<const float*>(src_base[s] + kQRowBytes)));
        if (lane == 0 && pending_store) bulk_wait_source_free<0>();
        __syncwarp();
#pragma unroll 1
        for (int j = 0; j < 6; j++) {
          const int p = lane + 32 * j;
          float acc[32];
          zero32(acc);
#pragma unroll
          for (int s = 0; s < P; s++) {
            uint4 q;
            uint32_t sf2;
            if (PULL) {
              q = *reinterpret_cast<const uint4*>(src_base[s] + 16 * p);
              sf2 = *reinterpret_cast<const unsigned short*>(src_base[s] + kValueBytes + 2 * p);
            } else {
              q = __ldcg(reinterpret_cast<const uint4*>(src_base[s] + 16 * p));
              sf2 = __ldcg(reinterpret_cast<const unsigned short*>(src_base[s] + kValueBytes + 2 * p));
            }
            perm4(q.x, q.y, q.z, q.w, f);
            const F2 e = e4m3_unpack2(sf2);
            const float s0 = __fmul_rn(e.lo, rsv[s]), s1 = __fmul_rn(e.hi, rsv[s]);
            const F2 sa = f2_splat((f & 2) ? s1 : s0), sb = f2_splat((f & 2) ? s0 : s1);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
              F2 v[4];
              e2m1_unpack8(w[k], v);
#pragma unroll
              for (int i = 0; i < 4; i++) {
                F2 a; a.lo = acc[8 * k + 2 * i]; a.hi = acc[8 * k + 2 * i + 1];
                a = f2_fma(v[i], k < 2 ? sa : sb, a);
                acc[8 * k + 2 * i] = a.lo; acc[8 * k + 2 * i + 1] = a.hi;
              }
            }
          }
          uint4 o[4];
          pack32_bf16(acc, o);
#pragma unroll
          for (int k = 0; k < 4; k++) sts16(obuf + p * 64 + ((k ^ f) << 4), o[k]);
        }
        fence_smem_to_async();
        __syncwarp();
        if (lane == 0) { bulk_store(io.out + (size_t)row * kRowB, obuf, kRowB); bulk_commit(); }
        pending_store = true;
      }
    }
    __syncwarp();
  }
  if (lane == 0 && pending_store) bulk_wait_done<0>();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (*err_word && atomicCAS(&io.status->code, 0u, (uint32_t)kStatusLoadTimeout) == 0u) {
      io.status->detail = 4u; io.status->cta = (uint32_t)cta; io.status->call = gen;
    }
    // the last CTA of this rank to leave advances the generation
    __threadfence();
    const uint32_t ticket = atomicAdd(ctrl + 1, 1u);
    if (ticket == (uint32_t)prm.ctas_per_rank - 1u) {
      ctrl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(ctrl) = gen + 1u;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Two-shot by pull (variant 3) and pull reduce-scatter + push all-gather (variant 4).
// Tile t = rows 4t .. 4t+3, one warp per row.  Iteration of a CTA: (1) encode the tile's rows into the own window
// and publish the tile flag; (2) the warp whose row this rank owns waits for every peer's tile flag, pulls their
// records of that row, sums in rank order, re-encodes, hands the re-encoding out (own window or every peer's) and
// sets the row flag; (3) the other warps wait for their row's flag and decode the owner's re-encoding.  Step (2) of
// tile t needs only step (1) of tile t of every rank, step (3) only step (2): no cycle of waits.
// Slot use inside buffer `gen & 1` of a window: (src = own rank, row) holds the own encoding; the owner's
// re-encoding of row r goes to slot ((owner + 1) % P, r) of the OWNER's window (variant 3) or to slot (owner, r)
// of every peer's window (variant 4); none of these slots is used for anything else by these two variants.
// ---------------------------------------------------------------------------------------------
template <int P, int AGPUSH>
__global__ void __launch_bounds__(kCmpWarps * 32, 1) cmp_ts_kernel(const __grid_constant__ CmpParams prm) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int f = (lane >> 1) & 3;
  const int local = blockIdx.x / prm.ctas_per_rank, cta = blockIdx.x - local * prm.ctas_per_rank;
  const CmpRank io = prm.io[local];
  const int me = io.rank;
  uint8_t* base = smem + (size_t)warp * kCmpWarpBytes;
  uint8_t* xbuf = base;
  uint8_t* recs = base + kRowB;
  uint8_t* obuf = base + 3 * kRowB;
  uint64_t* bar = reinterpret_cast<uint64_t*>(base + 4 * kRowB);
  uint32_t* err_word = reinterpret_cast<uint32_t*>(smem + (size_t)kCmpWarps * kCmpWarpBytes);
  if (lane == 0) { mbar_init(bar, 1); mbar_init(bar + 1, 1); }
  if (threadIdx.x == 0) *err_word = 0u;
  mbar_init_fence();
  __syncthreads();

  char* my_win = prm.win[me];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(my_win + cmp_ctrl_offset(P, prm.cap, prm.ntiles_cap));
  const uint32_t gen = *reinterpret_cast<volatile uint32_t*>(ctrl);
  const uint32_t want = gen + 1u;
  const size_t buf_rec = (size_t)(gen & 1u) * P * prm.cap * kRecStride;
  const size_t buf_flag = cmp_flags_offset(P, prm.cap) + (size_t)(gen & 1u) * P * prm.ntiles_cap * 4;
  const size_t buf_rowflag = cmp_rowflag_offset(P, prm.cap, prm.ntiles_cap) + (size_t)(gen & 1u) * prm.cap * 4;
  const int ntiles = (prm.rows + kCmpWarps - 1) / kCmpWarps;
  auto slot = [&](int src, int row) -> size_t { return buf_rec + ((size_t)src * prm.cap + row) * kRecStride; };

  auto wait_flag = [&](const uint32_t* fl, int row, int src, uint32_t detail) -> bool {
    bool ok = true;
    if (ld_acquire_sys(fl) != want) {
      const unsigned long long t0 = global_timer_ns();
      uint32_t n = 0;
      while (ld_acquire_sys(fl) != want) {
        if ((++n & 63u) == 0u && global_timer_ns() - t0 > prm.timeout_ns) {
          if (lane == 0) {
            if (atomicCAS(&io.status->code, 0u, (uint32_t)kStatusPeerTimeout) == 0u) {
              io.status->row = (uint32_t)row; io.status->source = (uint32_t)src; io.status->detail = detail;
              io.status->cta = (uint32_t)cta; io.status->call = gen;
            }
            atomicAdd(&io.status->count, 1u);
          }
          ok = false;
          break;
        }
      }
    }
    return __all_sync(0xffffffffu, ok);
  };
  // acc (slot order) += decode of pair p of the record at `rec` (shared or global memory, plain loads)
  auto add_pair = [&](float* acc, const uint8_t* rec, int p, float rs) {
    uint4 q = *reinterpret_cast<const uint4*>(rec + 16 * p);
    const uint32_t sf2 = *reinterpret_cast<const unsigned short*>(rec + kValueBytes + 2 * p);
    perm4(q.x, q.y, q.z, q.w, f);
    const F2 e = e4m3_unpack2(sf2);
    const float s0 = __fmul_rn(e.lo, rs), s1 = __fmul_rn(e.hi, rs);
    const F2 sa = f2_splat((f & 2) ? s1 : s0), sb = f2_splat((f & 2) ? s0 : s1);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
      F2 v[4];
      e2m1_unpack8(w[k], v);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        F2 a; a.lo = acc[8 * k + 2 * i]; a.hi = acc[8 * k + 2 * i + 1];
        a = f2_fma(v[i], k < 2 ? sa : sb, a);
        acc[8 * k + 2 * i] = a.lo; acc[8 * k + 2 * i + 1] = a.hi;
      }
    }
  };
  auto stage_out_pair = [&](const float* acc, int p) {
    uint4 o[4];
    pack32_bf16(acc, o);
#pragma unroll
    for (int k = 0; k < 4; k++) sts16(obuf + p * 64 + ((k ^ f) << 4), o[k]);
  };

  uint32_t xphase = 0, rphase = 0;
  bool pending_store = false;
  for (int t = cta; t < ntiles; t += prm.ctas_per_rank) {
    const int row = t * kCmpWarps + warp;
    const bool live = row < prm.rows;
    // ---------------------------------------------------------------- (1) encode into the own window, publish the tile
    if (live) {
      if (lane == 0) { mbar_arrive_expect(bar, kRowB); bulk_load(xbuf, io.x + (size_t)row * kRowB, kRowB, bar); }
      wait_row(bar, xphase & 1u, err_word);
      xphase++;
      char* rec = my_win + slot(me, row);
      float rs;
      encode_row_from_smem(xbuf, lane, 0.0f, false, rs,
                           [&](int p, uint4 q) { *reinterpret_cast<uint4*>(rec + 16 * p) = q; },
                           [&](int p, uint32_t sf2) { *reinterpret_cast<uint16_t*>(rec + kValueBytes + 2 * p) = (uint16_t)sf2; });
      if (lane == 0) {
        const uint32_t b = __float_as_uint(rs);
        *reinterpret_cast<uint4*>(rec + kQRowBytes) = make_uint4(b, b, b, b);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(reinterpret_cast<uint32_t*>(my_win + buf_flag) + (size_t)me * prm.ntiles_cap + t, want);
    if (live) {
      const int owner = row % P;
      if (lane == 0 && pending_store) bulk_wait_source_free<0>();   // obuf is free again
      __syncwarp();
      if (owner == me) {
        // ------------------------------------------------------------ (2) owner: pull, reduce, re-encode, hand out
        bool ok = true;
#pragma unroll 1
        for (int s = 0; s < P && ok; s++) {
          if (s == me) continue;
          ok = wait_flag(reinterpret_cast<const uint32_t*>(prm.win[s] + buf_flag) + (size_t)s * prm.ntiles_cap + t, row, s, 2u);
        }
        if (ok) {
          __syncwarp();
          if (lane == 0) {
            asm volatile("fence.proxy.async.global;" ::: "memory");
            mbar_arrive_expect(bar + 1, (uint32_t)(P * kRecPayload));
#pragma unroll
            for (int s = 0; s < P; s++) {
              uint8_t* dst = (s < 6 ? recs + s * kRecStride : xbuf + (s - 6) * kRecStride);
              bulk_load(dst, prm.win[s] + slot(s, row), kRecPayload, bar + 1);
            }
          }
          wait_row(bar + 1, rphase & 1u, err_word);
          rphase++;
          const uint8_t* srec[P];
          float rsv[P];
#pragma unroll
          for (int s = 0; s < P; s++) {
            srec[s] = s < 6 ? recs + s * kRecStride : xbuf + (s - 6) * kRecStride;
            rsv[s] = *reinterpret_cast<const float*>(srec[s] + kQRowBytes);
          }
          float am = 0.0f;
#pragma unroll 1
          for (int j = 0; j < 6; j++) {
            float acc[32];
            zero32(acc);
#pragma unroll
            for (int s = 0; s < P; s++) add_pair(acc, srec[s], lane + 32 * j, rsv[s]);
            am = absmax32(acc, am);
          }
          const RowScale sc2 = row_scale_from_amax(warp_max(am));
          // destinations of the re-encoding
          char* dst[P];
          int ndst = 0;
          if (AGPUSH) {
#pragma unroll
            for (int d = 0; d < P; d++) if (d != me) dst[ndst++] = prm.win[d] + slot(me, row);
          } else {
            dst[ndst++] = my_win + slot((me + 1) % P, row);
          }
#pragma unroll 1
          for (int j = 0; j < 6; j++) {
            const int p = lane + 32 * j;
            float acc[32];
            zero32(acc);
#pragma unroll
            for (int s = 0; s < P; s++) add_pair(acc, srec[s], p, rsv[s]);
            uint4 q;
            uint32_t sf2 = encode_pair_f32<true>(acc, [&](float b0, float b1, float& m0, float& m1) {
              return pair_block_scales(b0, b1, sc2.inv, m0, m1);
            }, q);                                                   // slot order in, slot order out
            zero32(acc);
            {
              const F2 e = e4m3_unpack2(sf2);
              const F2 sa = f2_splat(__fmul_rn(e.lo, sc2.rs)), sb = f2_splat(__fmul_rn(e.hi, sc2.rs));
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int k = 0; k < 4; k++) {
                F2 v[4];
                e2m1_unpack8(w[k], v);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                  F2 a; a.lo = 0.0f; a.hi = 0.0f;
                  a = f2_fma(v[i], k < 2 ? sa : sb, a);
                  acc[8 * k + 2 * i] = a.lo; acc[8 * k + 2 * i + 1] = a.hi;
                }
              }
            }
            stage_out_pair(acc, p);
            perm4(q.x, q.y, q.z, q.w, f);                            // back to canonical order for the wire
            if (f & 2) sf2 = ((sf2 & 0xffu) << 8) | (sf2 >> 8);
            for (int d = 0; d < ndst; d++) {
              *reinterpret_cast<uint4*>(dst[d] + 16 * p) = q;
              *reinterpret_cast<uint16_t*>(dst[d] + kValueBytes + 2 * p) = (uint16_t)sf2;
            }
          }
          if (lane == 0) {
            const uint32_t b = __float_as_uint(sc2.rs);
            for (int d = 0; d < ndst; d++) *reinterpret_cast<uint4*>(dst[d] + kQRowBytes) = make_uint4(b, b, b, b);
          }
          __syncwarp();                                              // the warp's stores happen-before the release below
          if (AGPUSH) {
            if (lane < P && lane != me) st_release_sys(reinterpret_cast<uint32_t*>(prm.win[lane] + buf_rowflag) + row, want);
          } else {
            if (lane == 0) st_release_sys(reinterpret_cast<uint32_t*>(my_win + buf_rowflag) + row, want);
          }
          fence_smem_to_async();
          __syncwarp();
          if (lane == 0) { bulk_store(io.out + (size_t)row * kRowB, obuf, kRowB); bulk_commit(); }
          pending_store = true;
        }
      } else {
        // ------------------------------------------------------------ (3) a peer owns the row: take its re-encoding
        const char* flag_win = AGPUSH ? my_win : prm.win[owner];
        if (wait_flag(reinterpret_cast<const uint32_t*>(flag_win + buf_rowflag) + row, row, owner, 3u)) {
          const uint8_t* rec;
          if (AGPUSH) {
            rec = reinterpret_cast<const uint8_t*>(my_win + slot(owner, row));     // local memory, written by the owner
          } else {
            __syncwarp();
            if (lane == 0) {
              asm volatile("fence.proxy.async.global;" ::: "memory");
              mbar_arrive_expect(bar + 1, (uint32_t)kRecPayload);
              bulk_load(recs, prm.win[owner] + slot((owner + 1) % P, row), kRecPayload, bar + 1);
            }
            wait_row(bar + 1, rphase & 1u, err_word);
            rphase++;
            rec = recs;
          }
          const float rs = AGPUSH ? __ldcg(reinterpret_cast<const float*>(rec + kQRowBytes))
                                  : *reinterpret_cast<const float*>(rec + kQRowBytes);
#pragma unroll 1
          for (int j = 0; j < 6; j++) {
            const int p = lane + 32 * j;
            float acc[32];
            zero32(acc);
            if (AGPUSH) {
              uint4 q = __ldcg(reinterpret_cast<const uint4*>(rec + 16 * p));
              const uint32_t sf2 = __ldcg(reinterpret_cast<const unsigned short*>(rec + kValueBytes + 2 * p));
              perm4(q.x, q.y, q.z, q.w, f);
              const F2 e = e4m3_unpack2(sf2);
              const float s0 = __fmul_rn(e.lo, rs), s1 = __fmul_rn(e.hi, rs);
              const F2 sa = f2_splat((f & 2) ? s1 : s0), sb = f2_splat((f & 2) ? s0 : s1);
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int k = 0; k < 4; k++) {
                F2 v[4];
                e2m1_unpack8(w[k], v);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                  F2 a; a.lo = 0.0f; a.hi = 0.0f;
                  a = f2_fma(v[i], k < 2 ? sa : sb, a);
                  acc[8 * k + 2 * i] = a.lo; acc[8 * k + 2 * i + 1] = a.hi;
                }
              }
            } else {
              add_pair(acc, rec, p, rs);
            }
            stage_out_pair(acc, p);
          }
          fence_smem_to_async();
          __syncwarp();
          if (lane == 0) { bulk_store(io.out + (size_t)row * kRowB, obuf, kRowB); bulk_commit(); }
          pending_store = true;
        }
      }
    }
    __syncwarp();
  }
  if (lane == 0 && pending_store) bulk_wait_done<0>();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (*err_word && atomicCAS(&io.status->code, 0u, (uint32_t)kStatusLoadTimeout) == 0u) {
      io.status->detail = 4u; io.status->cta = (uint32_t)cta; io.status->call = gen;
    }
    __threadfence();
    const uint32_t ticket = atomicAdd(ctrl + 1, 1u);
    if (ticket == (uint32_t)prm.ctas_per_rank - 1u) {
      ctrl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(ctrl) = gen + 1u;
    }
  }
}

using CmpFn = void (*)(const CmpParams);
static CmpFn cmp_find(int P, int variant) {
#define FP4AR_CMP(PP)                                             \
  if (P == PP) {                                                  \
    switch (variant) {                                            \
      case 0: return (CmpFn)cmp_kernel<PP, 0, 0>;                 \
      case 1: return (CmpFn)cmp_kernel<PP, 1, 0>;                 \
      case 2: return (CmpFn)cmp_kernel<PP, 1, 1>;                 \
      case 3: return (CmpFn)cmp_ts_kernel<PP, 0>;                 \
      case 4: return (CmpFn)cmp_ts_kernel<PP, 1>;                 \
    }                                                             \
  }
  FP4AR_CMP(1) FP4AR_CMP(2) FP4AR_CMP(4) FP4AR_CMP(8)
#undef FP4AR_CMP
  return nullptr;
}

}  // namespace fp4ar

using namespace fp4ar;

extern "C" size_t fp4ar_compare_window_bytes(int max_rows, int nranks) {
  if (max_rows < 1 || nranks < 1 || nranks > FP4AR_MAX_RANKS) return 0;
  const int ntiles = (max_rows + kCmpWarps - 1) / kCmpWarps;
  return cmp_rowflag_offset(nranks, max_rows, ntiles) + (((size_t)2 * max_rows * 4 + 255) & ~(size_t)255);
}

extern "C" int fp4ar_compare_allreduce(int variant, int rank, int nranks, int nlocal, void* const* windows, size_t window_bytes,
                                       int max_rows, const void* const* x, void* const* out, int rows, const float* gs,
                                       fp4ar_status_words* const* status, int timeout_ms, fp4ar_stream stream) {
  if (variant < 0 || variant > 4 || nranks < 1 || nranks > FP4AR_MAX_RANKS || !windows || !x || !out || !status)
    return FP4AR_ERR_ARGUMENT;
  if (!(nlocal == 1 || nlocal == nranks) || rows < 0 || rows > max_rows || timeout_ms < 1) return FP4AR_ERR_ARGUMENT;
  if (nlocal == 1 && (rank < 0 || rank >= nranks)) return FP4AR_ERR_ARGUMENT;
  if (window_bytes < fp4ar_compare_window_bytes(max_rows, nranks)) return FP4AR_ERR_ARGUMENT;
  CmpFn fn = cmp_find(nranks, variant);
  if (!fn) return FP4AR_ERR_UNSUPPORTED;
  CmpParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < nranks; r++) {
    if (!windows[r] || ((uintptr_t)windows[r] & 255)) return FP4AR_ERR_ARGUMENT;
    p.win[r] = (char*)windows[r];
  }
  for (int l = 0; l < nlocal; l++) {
    if (!x[l] || !out[l] || !status[l] || (((uintptr_t)x[l] | (uintptr_t)out[l]) & 15)) return FP4AR_ERR_ARGUMENT;
    p.io[l].x = (const char*)x[l]; p.io[l].out = (char*)out[l];
    p.io[l].status = reinterpret_cast<StatusWords*>(status[l]);
    p.io[l].rank = nlocal == 1 ? rank : l;
  }
  if (variant == 2) {
    if (!gs) return FP4AR_ERR_ARGUMENT;
    for (int r = 0; r < nranks; r++) {
      if (!(gs[r] > 0.0f)) return FP4AR_ERR_ARGUMENT;
      p.gs[r] = gs[r];
    }
  }
  p.rows = rows; p.cap = max_rows; p.ntiles_cap = (max_rows + kCmpWarps - 1) / kCmpWarps; p.nranks = nranks;
  p.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
  const int sms = device_sm_count();
  p.ctas_per_rank = nlocal == 1 ? sms : sms / nranks;
  if (p.ctas_per_rank < 1) return FP4AR_ERR_UNSUPPORTED;
  if (cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kCmpSmem) != cudaSuccess) return cuda_fail();
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(p.ctas_per_rank * nlocal), 1, 1);
  cfg.blockDim = dim3(kCmpWarps * 32, 1, 1);
  cfg.dynamicSmemBytes = kCmpSmem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  // emulated ranks wait on one another inside one launch: all CTAs must be resident together
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = nlocal > 1 ? 1 : 0;
  cfg.attrs = attr; cfg.numAttrs = 1;
  void* args[1] = {&p};
  if (cudaLaunchKernelExC(&cfg, (const void*)fn, args) != cudaSuccess) return cuda_fail();
  return FP4AR_OK;
}
