// The fused NVFP4 AllReduce kernel for sm_100a: encode -> push into the peers' receive windows over
// NVLink (bulk stores to peer-mapped addresses, 256 B packets) -> Lamport-in-data wait -> FP32
// rank-ordered decode-sum -> optional residual add + Gemma RMSNorm with BF16 / NVFP4 / MXFP8 output.
// One template covers tensor-parallel degree P = 1, 2, 4, 8, the one-shot algorithm and the two-shot
// algorithm (row owner = row % P reduces, re-encodes and broadcasts), and three input kinds (BF16
// rows, local NVFP4 rows with a static per-rank scale, NVFP4 rows that a producer kernel already
// pushed into the windows).
//
// What the reference project does for the same job, for comparison: kernels/push/tp2_l2.cu:744-950
// (TP2 one-shot), kernels/push/tp4_l4.cu:285-676 (TP4 two-shot), kernels/fused_norm/lnorm.cu:566-697
// (TP2 + norm).  This kernel is organised differently:
//   * A team of T warps walks its rows as a software pipeline: step k runs (two-shot) the owner step
//     of row k - lag_owner, encodes and pushes row k, and finishes row k - lag_finish, so that peer data
//     has whole steps to arrive before it is needed (one-shot: lag_finish = 1).  All ranks walk the
//     same rows in the same order, so the waits cannot form a cycle.
//   * A receive slot is re-armed (overwritten with sentinels) by the team that consumed it, in the same
//     call, while the line is still in L2.  At every call boundary the whole window is sentinel again,
//     so two buffers (call parity) suffice, one-shot and two-shot share the same memory, and there is
//     no per-call "what did the previous call use" state.
//   * Inside a lane the four 16-byte chunks of a 32-value pair are kept in a lane-dependent order
//     (slot k holds chunk k ^ ((lane >> 1) & 3)), so that every 64-byte-per-lane shared-memory access
//     is bank-conflict free with static register indices; only the compact 16 B of E2M1 per pair is
//     permuted, with 8 selects.
//   * Input rows enter shared memory by bulk asynchronous copies; outputs and records leave through
//     staging rows and one bulk store each.  The residual row of the norm epilogue goes global ->
//     registers -> global (every lane owns whole 64-byte pieces).
//   * Every wait is bounded (see fp4ar_async.cuh).
#pragma once
#include "../include/fp4ar_codec.cuh"
#include "../include/fp4ar_async.cuh"

namespace fp4ar {

constexpr int kRowBytes = kHidden * 2;   // 12288: one BF16 row
constexpr int kMaxRanks = 8;

enum : int { kFlagXport = 1, kFlagLoopback = 2 };

struct RankIO {
  const char* x;
  char* out;
  const char* res_in;
  char* res_out;
  char* outq;
  char* win[kMaxRanks];
  uint32_t* ctrl;        // per-CTA call counters
  StatusWords* status;
  uint32_t* poison;      // device-mapped host word: non-zero after a wait gave up (read by the launch path)
  int rank;
  int pad;
};

struct ArParams {
  RankIO io[kMaxRanks];  // one entry per rank run by this launch (1 in production)
  const char* weight;
  float gs[kMaxRanks];
  float eps, wbias, qscale;
  int rows, ctas_per_rank, flags;
  int cap, capo;
  unsigned long long buf_bytes, timeout_ns;
  int lag_owner, lag_finish;          // two-shot pipeline depths in steps (1 <= lag_owner < lag_finish <= 4)
  unsigned long long* phase_cycles;   // tuning builds only (-DFP4AR_PHASE_TIMERS): 16 per-phase cycle counters
};

template <int P, int ALGO, int IN, int EPI, int T>
struct ArShape {
  static constexpr int NJ = 6 / T;                                   // pairs per lane per row
  static constexpr bool kTwoShot = ALGO == 1 && P > 1;
  // Rows are finished LAG steps after they were encoded: 1 for one-shot (every source pushed during the previous
  // step), 2 for two-shot (the owner re-encodes and broadcasts during the step in between), so that a finishing
  // team finds its data in place and the ranks need not run in lock step.
  // The two-shot lags are run-time parameters (owner step lag_o >= 1 steps after the encode, finish lag_f > lag_o);
  // kMaxLag bounds them and sizes the record ring.
  static constexpr int kMaxLag = kTwoShot ? 4 : 1;
  static constexpr int NXB = IN == 0 ? 2 : 0;                        // x row buffers (the residual never sits in shared memory)
  static constexpr int NREC = (IN == 1 ? 2 : 1) + kMaxLag;
  static constexpr int kOutBytes = EPI <= 1 ? kRowBytes : (EPI == 2 ? 3584 : 6400);
  static constexpr int kMisc = 128;                                  // mbarriers + reduction scratch
  static constexpr int kTeamBytes = NXB * kRowBytes + kOutBytes + NREC * kRecStride + kMisc;
  static constexpr int kCtaExtra = kRecStride + 128 + 1024;          // sentinel record + abort flag + scale table
  static constexpr int NSG = IN == 2 ? P : P - 1;                    // sources read from the window
  // Two-shot owners hold a whole FP32 row slice in registers and the norm epilogue holds BF16 z and the
  // residual: those shapes get fewer, fatter threads.
  // (Register budget per thread = 65536 / (32 * T * kMaxTeams).)
  static constexpr int kHeavy = (ALGO == 1 || EPI > 0) ? 1 : 0;
  // Three-warp teams: 4 per CTA (heavy shapes) or 5; six-warp teams: 3 per CTA (18 warps at up to 112 registers; a
  // fourth team at 80 registers measured 20-30 % slower).
  static constexpr int kMaxTeams = T == 3 ? (kHeavy ? 4 : 5) : (T == 1 ? 8 : 3);
  static __host__ __device__ constexpr int smem_bytes(int teams) { return teams * kTeamBytes + kCtaExtra; }
};

// Conditional swaps that take chunk order to slot order and back (the permutation is an involution).
__device__ __forceinline__ void lane_permute4(uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d, int f) {
  if (f & 1) { uint32_t t = a; a = b; b = t; t = c; c = d; d = t; }
  if (f & 2) { uint32_t t = a; a = c; c = t; t = b; b = d; d = t; }
}

// acc (slot order) += decode of four slot-ordered value words with the scales of slots {0,1} and {2,3}.
__device__ __forceinline__ void decode_acc_slots(float* acc, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,
                                                 float sa, float sb) {
  const F2 s01 = f2_splat(sa), s23 = f2_splat(sb);
  const uint32_t w[4] = {w0, w1, w2, w3};
#pragma unroll
  for (int k = 0; k < 4; k++) {
    F2 v[4];
    e2m1_unpack8(w[k], v);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      F2 a; a.lo = acc[8 * k + 2 * i]; a.hi = acc[8 * k + 2 * i + 1];
      a = f2_fma(v[i], k < 2 ? s01 : s23, a);
      acc[8 * k + 2 * i] = a.lo; acc[8 * k + 2 * i + 1] = a.hi;
    }
  }
}
// One source: canonical (q, sf2, rs) -> slot order -> accumulate.
__device__ __forceinline__ void decode_acc_lane(float* acc, uint4 q, uint32_t sf2, float rs, int f) {
  lane_permute4(q.x, q.y, q.z, q.w, f);
  const F2 e = e4m3_unpack2(sf2);
  const float s0 = __fmul_rn(e.lo, rs), s1 = __fmul_rn(e.hi, rs);
  decode_acc_slots(acc, q.x, q.y, q.z, q.w, (f & 2) ? s1 : s0, (f & 2) ? s0 : s1);
}

// Per-phase cycle counters for tuning builds (-DFP4AR_PHASE_TIMERS); absent from the production library.
#ifdef FP4AR_PHASE_TIMERS
#define FP4AR_PHASE(idx)                                                               \
  do {                                                                                 \
    if (leader && team == 0) {                                                         \
      const long long now_ = clock64();                                                \
      atomicAdd(&prm.phase_cycles[idx], (unsigned long long)(now_ - phase_t0_));         \
      phase_t0_ = now_;                                                                \
    }                                                                                  \
  } while (0)
#else
#define FP4AR_PHASE(idx) do { } while (0)
#endif

template <int T>
struct TeamSync {
  int bar_id;
  __device__ __forceinline__ void sync() const {
    if (T == 1) __syncwarp();
    else asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(32 * T) : "memory");
  }
};

template <int P, int ALGO, int IN, int EPI, int T>
__global__ void __launch_bounds__(32 * T * ArShape<P, ALGO, IN, EPI, T>::kMaxTeams, 1) ar_kernel(const __grid_constant__ ArParams prm) {
  using S = ArShape<P, ALGO, IN, EPI, T>;
  constexpr int NJ = S::NJ, NXB = S::NXB, NREC = S::NREC, NSG = S::NSG;
  constexpr bool kTwoShot = S::kTwoShot;
  constexpr int NXB1 = NXB > 0 ? NXB : 1;   // keeps index arithmetic well-formed in shapes without row buffers
  extern __shared__ __align__(1024) uint8_t smem[];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nteams = (blockDim.x >> 5) / T;
  const int team = warp / T, tw = warp % T;
  const bool leader = tw == 0 && lane == 0;
  const int f = (lane >> 1) & 3;
  const int G = prm.ctas_per_rank;
  const int lr = blockIdx.x / G, cta = blockIdx.x % G;
  const RankIO& io = prm.io[lr];
  const int me = io.rank;
  const bool xport = (prm.flags & kFlagXport) != 0;
  const bool loopb = (prm.flags & kFlagLoopback) != 0;

  // ---- shared-memory carve-up ----
  uint8_t* tbase = smem + (size_t)team * S::kTeamBytes;
  uint8_t* xb = tbase;                                   // NXB buffers for BF16 input rows
  uint8_t* outst = tbase + NXB * kRowBytes;              // output staging row
  uint8_t* recs = outst + S::kOutBytes;                  // NREC encoded records
  uint64_t* xbar = reinterpret_cast<uint64_t*>(recs + NREC * kRecStride);  // [3] x loads
  uint64_t* qbar = xbar + 2;                             // [6] NVFP4 record loads
  float* red = reinterpret_cast<float*>(qbar + 6);       // [2][6] reduction exchange
  uint8_t* sentinel = smem + (size_t)nteams * S::kTeamBytes;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(sentinel + kRecStride);
  float2* scale_tab = reinterpret_cast<float2*>(sentinel + kRecStride + 128);
  const ScaleLut slut{scale_tab};
  const TeamSync<T> tsync{1 + team};

  // ---- prologue: nothing here touches global memory written by an earlier kernel ----
  if (threadIdx.x == 0) *abort_flag = 0u;
  if (leader) {
#pragma unroll
    for (int i = 0; i < 8; i++) mbar_init(xbar + i, 1);
  }
  for (int i = threadIdx.x; i < kRecStride / 16; i += blockDim.x) {
    uint4 v;
    if (i < kValueBytes / 16) v = make_uint4(kSentWord, kSentWord, kSentWord, kSentWord);
    else if (i < kQRowBytes / 16) v = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
    else if (i == kQRowBytes / 16) v = make_uint4(kSentRow, kSentRow, kSentRow, kSentRow);
    else v = make_uint4(0, 0, 0, 0);
    sts16(sentinel + 16 * i, v);
  }
  fill_scale_lut(scale_tab, threadIdx.x, blockDim.x);
  mbar_init_fence();
  fence_smem_to_async();
  __syncthreads();
  const int rb = (int)(((long long)cta * prm.rows) / G), re = (int)(((long long)(cta + 1) * prm.rows) / G);
  const int nk = (re - rb > team) ? (re - rb - team + nteams - 1) / nteams : 0;
  auto row_of = [&](int k) { return rb + team + nteams * k; };
  pdl_wait_prior_grids();
  // ---- first loads: they need nothing from the call state, so they go out before it is read ----
  if (leader && nk > 0) {
    if (IN == 0) {
      mbar_arrive_expect(xbar + 0, kRowBytes);
      bulk_load(xb, io.x + (size_t)row_of(0) * kRowBytes, kRowBytes, xbar + 0);
      if (nk > 1) {
        mbar_arrive_expect(xbar + 1, kRowBytes);
        bulk_load(xb + kRowBytes, io.x + (size_t)row_of(1) * kRowBytes, kRowBytes, xbar + 1);
      }
    } else if (IN == 1) {
      mbar_arrive_expect(qbar + 0, kQRowBytes);
      bulk_load(recs, io.x + (size_t)row_of(0) * kQRowBytes, kQRowBytes, qbar + 0);
    }
  }

  const uint32_t call = io.ctrl[cta];
  pdl_release_dependents();

  WaitCtx wctx;
  wctx.status = io.status; wctx.cta_abort = abort_flag; wctx.host_poison = io.poison; wctx.limit_ns = prm.timeout_ns;
  wctx.cta = (uint32_t)cta; wctx.call = call;

  const size_t buf_off = (size_t)(call & 1u) * prm.buf_bytes;
  char* const my_buf = io.win[me] + buf_off;
  const int cap = prm.cap, capo = prm.capo;
  auto os_slot = [&](int src, int row) -> size_t { return ((size_t)src * cap + row) * kRecStride; };
  auto rs_slot = [&](int src, int row) -> size_t { return ((size_t)src * capo + row / P) * kRecStride; };
  auto ag_slot = [&](int own, int row) -> size_t { return ((size_t)(P + own) * capo + row / P) * kRecStride; };

  int red_phase = 0;

  // Exchange one float per (warp, j) across the team: every lane returns with all six group values.
  auto team_gather6 = [&](const float* mine, float* all6) {
    float* slot = red + 6 * (red_phase & 1);
    red_phase++;
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < NJ; j++) slot[tw + T * j] = mine[j];
    }
    tsync.sync();
#pragma unroll
    for (int g = 0; g < 6; g++) all6[g] = slot[g];
  };

  // =============================================================================================
  // Row completion shared by every algorithm: `fill(j, acc)` produces the FP32 sum of pair j in slot
  // order; this routine applies the epilogue, stages the row and lets the leader store it.
  // `leader_extra()` issues the leader's other stores of this row (re-arm, broadcast).
  // =============================================================================================
  auto finish_row = [&](int row, auto&& fill, auto&& leader_extra) {
    const int pbase = tw;  // pair of (lane, j) = lane + 32 * (tw + T * j)
    if constexpr (EPI == 0) {
#pragma unroll
      for (int j = 0; j < NJ; j++) {
        const int p = lane + 32 * (pbase + T * j);
        float acc[32];
        fill(j, acc);
        uint4 o[4];
        pack32_bf16(acc, o);
#pragma unroll
        for (int k = 0; k < 4; k++) sts16(outst + p * 64 + ((k ^ f) << 4), o[k]);
      }
      fence_smem_to_async();
      tsync.sync();
      if (leader) {
        bulk_store(io.out + (size_t)row * kRowBytes, outst, kRowBytes);
        leader_extra();
      }
    } else {
      // The residual row is read straight from global memory into registers (issued before the window data is
      // polled and decoded, so its latency is hidden) and the updated residual is written straight back: each lane
      // touches whole 64-byte pieces, so every 32-byte sector it reads or writes is fully used.
      const char* res_row = io.res_in + (size_t)row * kRowBytes;
      char* res_out_row = io.res_out + (size_t)row * kRowBytes;
      uint4 rr[NJ][4];
#pragma unroll
      for (int j = 0; j < NJ; j++) {
        const int p = lane + 32 * (pbase + T * j);
#pragma unroll
        for (int k = 0; k < 4; k++) rr[j][k] = *reinterpret_cast<const uint4*>(res_row + p * 64 + ((k ^ f) << 4));
      }
      uint4 zb[NJ][4];
      float gsum[NJ];
#pragma unroll
      for (int j = 0; j < NJ; j++) {
        const int p = lane + 32 * (pbase + T * j);
        float acc[32];
        fill(j, acc);
        const float sp = add_residual_sumsq(acc, rr[j]);
        pack32_bf16(acc, zb[j]);
#pragma unroll
        for (int k = 0; k < 4; k++) *reinterpret_cast<uint4*>(res_out_row + p * 64 + ((k ^ f) << 4)) = zb[j][k];
        gsum[j] = warp_sum_butterfly(sp);
      }
      float g6[6];
      team_gather6(gsum, g6);   // also: every lane is done polling, so the slots may be re-armed
      if (leader) leader_extra();
      float ss = g6[0];
#pragma unroll
      for (int g = 1; g < 6; g++) ss = __fadd_rn(ss, g6[g]);
      const float rinv = norm_rinv(ss, prm.eps);
#pragma unroll
      for (int j = 0; j < NJ; j++) {
        const int p = lane + 32 * (pbase + T * j);
        uint4 wt[4];
#pragma unroll
        for (int k = 0; k < 4; k++) wt[k] = __ldg(reinterpret_cast<const uint4*>(prm.weight + p * 64 + ((k ^ f) << 4)));
        float y[32];
        norm_pair(zb[j], wt, rinv, prm.wbias, y);
        uint4 yb[4];
        pack32_bf16(y, yb);
        if (EPI == 1) {
#pragma unroll
          for (int k = 0; k < 4; k++) sts16(outst + p * 64 + ((k ^ f) << 4), yb[k]);
        } else if (EPI == 2) {
          uint4 q;
          uint32_t sf2 = quant_pair_nvfp4_out(yb, prm.qscale, q);   // slot order: bytes/words follow slots
          lane_permute4(q.x, q.y, q.z, q.w, f);
          if (f & 2) sf2 = ((sf2 & 0xffu) << 8) | (sf2 >> 8);
          sts16(outst + p * 16, q);
          *reinterpret_cast<uint16_t*>(outst + kValueBytes + 2 * p) = (uint16_t)sf2;
        } else {
          uint4 v[2];
          const uint32_t e = quant_pair_mxfp8_out(yb, v);            // v: slot k -> words 2k, 2k+1
          const uint32_t* vw = reinterpret_cast<const uint32_t*>(v);
#pragma unroll
          for (int k = 0; k < 4; k++)
            *reinterpret_cast<uint2*>(outst + p * 32 + ((k ^ f) << 3)) = make_uint2(vw[2 * k], vw[2 * k + 1]);
          outst[kHidden + p] = (uint8_t)e;
        }
      }
      fence_smem_to_async();
      tsync.sync();
      if (leader) {
        if (EPI == 1) bulk_store(io.out + (size_t)row * kRowBytes, outst, kRowBytes);
        else if (EPI == 2) bulk_store(io.outq + (size_t)row * kQRowBytes, outst, kQRowBytes);
        else bulk_store(io.outq + (size_t)row * kMxRowBytes, outst, kMxRowBytes);
      }
    }
  };

  // Poll one window record for pair p until its 16 value bytes and 2 scale bytes are sentinel-free.
  auto poll_pair = [&](const char* rec, int p, uint4& q, uint32_t& sf2, int row, int src, int phase) {
    q = poll_ld16(rec + 16 * p);
    sf2 = poll_ld2(rec + kValueBytes + 2 * p);
    if (values_pending(q) | scales_pending(sf2)) {
      const unsigned long long t0 = global_timer_ns();
      uint32_t n = 0;
      while (true) {
        if (*abort_flag) break;
        if (values_pending(q)) q = poll_ld16(rec + 16 * p);
        if (scales_pending(sf2)) sf2 = poll_ld2(rec + kValueBytes + 2 * p);
        if (!(values_pending(q) | scales_pending(sf2))) break;
        if ((++n & 127u) == 0u && global_timer_ns() - t0 > prm.timeout_ns) {
          report_wait_failure(wctx, kStatusPeerTimeout, (uint32_t)row, (uint32_t)src, (uint32_t)phase);
          break;
        }
      }
    }
  };
  auto poll_rowscale = [&](const char* rec, int row, int src, int phase) -> float {
    uint32_t b = poll_ld4(rec + kQRowBytes);
    if (rowscale_pending(b)) {
      const unsigned long long t0 = global_timer_ns();
      uint32_t n = 0;
      while (true) {
        if (*abort_flag) break;
        b = poll_ld4(rec + kQRowBytes);
        if (!rowscale_pending(b)) break;
        if ((++n & 127u) == 0u && global_timer_ns() - t0 > prm.timeout_ns) {
          report_wait_failure(wctx, kStatusPeerTimeout, (uint32_t)row, (uint32_t)src, (uint32_t)phase);
          break;
        }
      }
    }
    return __uint_as_float(b);
  };
  // i-th rank among the sources that live in the window
  auto window_source = [&](int i) { return IN == 2 ? i : i + (i >= me ? 1 : 0); };

  // =============================================================================================
  // main pipeline.  Step k: (two-shot) owner step of row k-lag_o; encode + push row k; finish row k-lag_f.
  // =============================================================================================
#ifdef FP4AR_PHASE_TIMERS
  long long phase_t0_ = clock64();
#endif
  constexpr int kPfSrc = NSG > 0 ? NSG : 1;
  constexpr bool kPfAll = NJ * NSG <= 8;            // a whole row of every window source fits in registers
  auto settle_rs = [&](uint32_t bits, const char* rec, int row, int src, int phase) -> float {
    return rowscale_pending(bits) ? poll_rowscale(rec, row, src, phase) : __uint_as_float(bits);
  };

  const int lag_o = kTwoShot ? prm.lag_owner : 0;
  const int lag_f = kTwoShot ? prm.lag_finish : 1;
  for (int k = 0; k < nk + lag_f; k++) {
    FP4AR_PHASE(0);
    if (leader) bulk_wait_source_free<0>();
    tsync.sync();
    FP4AR_PHASE(1);   // drain wait + barrier
    if (leader && IN == 1 && k + 1 < nk) {
      const int b = (k + 1) % NREC;
      mbar_arrive_expect(qbar + b, kQRowBytes);
      bulk_load(recs + b * kRecStride, io.x + (size_t)row_of(k + 1) * kQRowBytes, kQRowBytes, qbar + b);
    }

    // ------------------------------------------------------------------ early window loads
    // (a) the row finished in this step (k - lag_f): one-shot sources, or the owner's broadcast of a row owned by a peer;
    // (b) two-shot: the reduce-scatter sources of row k - lag_owner when this rank owns it (loaded in the owner step).
    // Everything was pushed at least one full step ago; stage-specific code validates and falls back to polling.
    const int kf = k - lag_f;                        // row index (in this team's sequence) finished in this step
    const bool fin = kf >= 0 && kf < nk;
    const int frow = fin ? row_of(kf) : 0;
    const bool fin_owned = kTwoShot && fin && (frow % P) == me;
    const char* fsrc[kTwoShot ? 1 : kPfSrc];
    uint32_t frs[kTwoShot ? 1 : kPfSrc];
    uint4 fq[NJ][kTwoShot ? 1 : (kPfAll ? kPfSrc : 1)];
    uint32_t fsf[NJ][kTwoShot ? 1 : (kPfAll ? kPfSrc : 1)];
    bool f_has_rs = false;
    if (fin) {
      if constexpr (!kTwoShot) {
#pragma unroll
        for (int i = 0; i < NSG; i++) fsrc[i] = my_buf + os_slot(window_source(i), frow);
        f_has_rs = IN == 0;
#pragma unroll
        for (int i = 0; i < NSG; i++)
          if (f_has_rs) frs[i] = poll_ld4(fsrc[i] + kQRowBytes);
        if (kPfAll) {
#pragma unroll
          for (int jj = 0; jj < NJ; jj++) {
            const int p = lane + 32 * (tw + T * jj);
#pragma unroll
            for (int i = 0; i < NSG; i++) {
              fq[jj][i] = poll_ld16(fsrc[i] + 16 * p);
              fsf[jj][i] = poll_ld2(fsrc[i] + kValueBytes + 2 * p);
            }
          }
        }
      } else if (!fin_owned) {
        fsrc[0] = my_buf + ag_slot(frow % P, frow);
        f_has_rs = !(loopb && IN >= 1);
        if (f_has_rs) frs[0] = poll_ld4(fsrc[0] + kQRowBytes);
#pragma unroll
        for (int jj = 0; jj < NJ; jj++) {
          const int p = lane + 32 * (tw + T * jj);
          fq[jj][0] = poll_ld16(fsrc[0] + 16 * p);
          fsf[jj][0] = poll_ld2(fsrc[0] + kValueBytes + 2 * p);
        }
      }
    }
    FP4AR_PHASE(2);   // early loads issued

    // ------------------------------------------------------------------ owner step of row k-lag_o (two-shot)
    // Reduce every source, re-encode into rec, broadcast.  The row is finished (decoded, epilogue) lag_finish -
    // lag_owner steps later like every other row, from the record kept in the ring.
    if constexpr (kTwoShot) {
      const int ko = k - lag_o;
      if (ko >= 0 && ko < nk && (row_of(ko) % P) == me) {
        const int row = row_of(ko);
        uint8_t* rec_own = recs + (ko % NREC) * kRecStride;
        const char* osrc[kPfSrc];
        float wrs[kPfSrc];
        uint32_t ors[kPfSrc];
#pragma unroll
        for (int i = 0; i < NSG; i++) {
          osrc[i] = my_buf + rs_slot(window_source(i), row);
          if (IN == 0) ors[i] = poll_ld4(osrc[i] + kQRowBytes);
        }
        uint4 oq[NJ][kPfAll ? kPfSrc : 1];
        uint32_t osf[NJ][kPfAll ? kPfSrc : 1];
        if (kPfAll) {
#pragma unroll
          for (int jj = 0; jj < NJ; jj++) {
            const int p = lane + 32 * (tw + T * jj);
#pragma unroll
            for (int i = 0; i < NSG; i++) {
              oq[jj][i] = poll_ld16(osrc[i] + 16 * p);
              osf[jj][i] = poll_ld2(osrc[i] + kValueBytes + 2 * p);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < NSG; i++) {
          const int s = window_source(i);
          wrs[i] = IN == 0 ? settle_rs(ors[i], osrc[i], row, s, 2) : prm.gs[s];
        }
        float own_rs = 0.0f;
        if (IN == 0) own_rs = *reinterpret_cast<const float*>(rec_own + kQRowBytes);
        if (IN == 1) own_rs = prm.gs[me];
        float sums[NJ][32];
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; j++) {
          const int p = lane + 32 * (tw + T * j);
          uint4 wq[kPfSrc];
          uint32_t wsf[kPfSrc];
#pragma unroll
          for (int i = 0; i < NSG; i++) {
            if (kPfAll) { wq[i] = oq[j][i]; wsf[i] = osf[j][i]; }
            else { wq[i] = poll_ld16(osrc[i] + 16 * p); wsf[i] = poll_ld2(osrc[i] + kValueBytes + 2 * p); }
          }
#pragma unroll
          for (int i = 0; i < NSG; i++)
            if (values_pending(wq[i]) | scales_pending(wsf[i])) poll_pair(osrc[i], p, wq[i], wsf[i], row, window_source(i), 2);
          zero32(sums[j]);
          if (!xport) {
#pragma unroll
            for (int i = 0; i <= NSG; i++) {
              if (IN != 2 && i == me) {
                const uint4 q = lds16(rec_own + 16 * p);
                const uint32_t sf2 = *reinterpret_cast<const uint16_t*>(rec_own + kValueBytes + 2 * p);
                decode_acc_lane(sums[j], q, sf2, own_rs, f);
              }
              if (i < NSG) decode_acc_lane(sums[j], wq[i], wsf[i], wrs[i], f);
            }
            am = absmax32(sums[j], am);
          }
        }
        am = warp_max(am);
        {
          float mine[NJ], g6[6];
#pragma unroll
          for (int j = 0; j < NJ; j++) mine[j] = am;
          team_gather6(mine, g6);   // also orders every lane's reads of rec_own before the rewrite below
#pragma unroll
          for (int g = 0; g < 6; g++) am = fmaxf(am, g6[g]);
        }
        const RowScale sc = row_scale_from_amax(am);
        const bool lut_ok = scale_lut_range_ok(sc.inv);
        if (!xport) {
#pragma unroll
          for (int j = 0; j < NJ; j++) {
            const int p = lane + 32 * (tw + T * j);
            uint4 q;
            uint32_t sf2 = encode_pair_f32<true>(sums[j], [&](float b0, float b1, float& m0, float& m1) {
              return pair_block_scales_lut(b0, b1, sc.inv, slut, lut_ok, m0, m1);
            }, q);   // slot order
            lane_permute4(q.x, q.y, q.z, q.w, f);
            if (f & 2) sf2 = ((sf2 & 0xffu) << 8) | (sf2 >> 8);
            sts16(rec_own + 16 * p, q);
            *reinterpret_cast<uint16_t*>(rec_own + kValueBytes + 2 * p) = (uint16_t)sf2;
          }
          if (leader) {
            const uint32_t rb4 = __float_as_uint(sc.rs);
            sts16(rec_own + kQRowBytes, make_uint4(rb4, rb4, rb4, rb4));
          }
        } else {
          if (IN == 2) {
#pragma unroll
            for (int j = 0; j < NJ; j++) {
              const int p = lane + 32 * (tw + T * j);
              sts16(rec_own + 16 * p, make_uint4(0x11111111u, 0x11111111u, 0x11111111u, 0x11111111u));
              *reinterpret_cast<uint16_t*>(rec_own + kValueBytes + 2 * p) = (uint16_t)0x3838u;
            }
          }
          if (leader) sts16(rec_own + kQRowBytes, make_uint4(0x3f800000u, 0x3f800000u, 0x3f800000u, 0x3f800000u));
        }
        fence_smem_to_async();
        tsync.sync();
        if (leader) {
#pragma unroll
          for (int d = 0; d < P; d++) {
            if (d == me) continue;
            char* dst = (loopb ? my_buf : io.win[d] + buf_off) + ag_slot(me, row);
            bulk_store(dst, rec_own, kRecPayload);
          }
#pragma unroll
          for (int i = 0; i < NSG; i++) bulk_store(const_cast<char*>(osrc[i]), sentinel, kRecPayload);
        }
      }
    }
    FP4AR_PHASE(3);   // owner step

    // ------------------------------------------------------------------ stage A: encode + push row k
    if (k < nk) {
      const int row = row_of(k);
      uint8_t* rec = recs + (k % NREC) * kRecStride;
      if (IN == 0) {
        const int b = k % NXB1;
        const uint8_t* xrow = xb + b * kRowBytes;
        mbar_wait_bounded(xbar + b, (uint32_t)((k / NXB1) & 1), wctx, row);
        FP4AR_PHASE(4);   // wait for x
        if (!xport) {
          uint32_t bmp[NJ];
          float am = 0.0f;
#pragma unroll
          for (int j = 0; j < NJ; j++) {
            const int p = lane + 32 * (tw + T * j);
            const __nv_bfloat162 z2 = __floats2bfloat162_rn(0.0f, 0.0f);
            __nv_bfloat162 ma = z2, mb = z2;
            ma = chunk_absmax(lds16(xrow + p * 64 + ((0 ^ f) << 4)), ma);
            ma = chunk_absmax(lds16(xrow + p * 64 + ((1 ^ f) << 4)), ma);
            mb = chunk_absmax(lds16(xrow + p * 64 + ((2 ^ f) << 4)), mb);
            mb = chunk_absmax(lds16(xrow + p * 64 + ((3 ^ f) << 4)), mb);
            const uint32_t xa = bf16x2_hmax_bits(ma), xbm = bf16x2_hmax_bits(mb);   // slots {0,1} / {2,3}
            bmp[j] = (f & 2) ? (xbm | (xa << 16)) : (xa | (xbm << 16));            // low half = block 0
            am = fmaxf(am, __uint_as_float(max(xa, xbm) << 16));
          }
          am = warp_max(am);
          if (T > 1) {
            float mine[NJ], g6[6];
#pragma unroll
            for (int j = 0; j < NJ; j++) mine[j] = am;
            team_gather6(mine, g6);
#pragma unroll
            for (int g = 0; g < 6; g++) am = fmaxf(am, g6[g]);
          }
          const RowScale sc = row_scale_from_amax(am);
          const bool lut_ok = scale_lut_range_ok(sc.inv);
          FP4AR_PHASE(5);   // amax pass + exchange
#pragma unroll
          for (int j = 0; j < NJ; j++) {
            const int p = lane + 32 * (tw + T * j);
            const float bm0 = __uint_as_float(bmp[j] << 16), bm1 = __uint_as_float(bmp[j] & 0xffff0000u);
            float m0, m1;
            const uint32_t sf2 = pair_block_scales_lut(bm0, bm1, sc.inv, slut, lut_ok, m0, m1);
            const float mlo = (f & 2) ? m1 : m0, mhi = (f & 2) ? m0 : m1;
            uint32_t w0 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((0 ^ f) << 4)), mlo);
            uint32_t w1 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((1 ^ f) << 4)), mlo);
            uint32_t w2 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((2 ^ f) << 4)), mhi);
            uint32_t w3 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((3 ^ f) << 4)), mhi);
            lane_permute4(w0, w1, w2, w3, f);
            sts16(rec + 16 * p, make_uint4(w0, w1, w2, w3));
            *reinterpret_cast<uint16_t*>(rec + kValueBytes + 2 * p) = (uint16_t)sf2;
          }
          if (leader) {
            const uint32_t rb4 = __float_as_uint(sc.rs);
            sts16(rec + kQRowBytes, make_uint4(rb4, rb4, rb4, rb4));
          }
        } else {
          // transport-only mode: a fixed payload that contains no sentinel
#pragma unroll
          for (int j = 0; j < NJ; j++) {
            const int p = lane + 32 * (tw + T * j);
            sts16(rec + 16 * p, make_uint4(0x11111111u, 0x11111111u, 0x11111111u, 0x11111111u));
            *reinterpret_cast<uint16_t*>(rec + kValueBytes + 2 * p) = (uint16_t)0x3838u;
          }
          if (leader) sts16(rec + kQRowBytes, make_uint4(0x3f800000u, 0x3f800000u, 0x3f800000u, 0x3f800000u));
        }
        fence_smem_to_async();
        tsync.sync();
      } else if (IN == 1) {
        mbar_wait_bounded(qbar + (k % NREC), (uint32_t)((k / NREC) & 1), wctx, row);
      }

      if (leader) {
        if (IN != 2) {
          const uint32_t bytes = IN == 0 ? (uint32_t)kRecPayload : (uint32_t)kQRowBytes;
          if (!kTwoShot) {
#pragma unroll
            for (int d = 0; d < P; d++) {
              if (d == me) continue;
              char* dst = loopb ? my_buf + os_slot(d, row) : io.win[d] + buf_off + os_slot(me, row);
              bulk_store(dst, rec, bytes);
            }
          } else {
            const int owner = row % P;
            if (owner != me) {
              char* dst = loopb ? my_buf + ag_slot(owner, row) : io.win[owner] + buf_off + rs_slot(me, row);
              bulk_store(dst, rec, bytes);
            } else if (loopb) {
#pragma unroll
              for (int s = 0; s < P; s++)
                if (s != me) bulk_store(my_buf + rs_slot(s, row), rec, bytes);
            }
          }
        }
        if (IN == 0 && k + 2 < nk) {
          const int b = k % NXB1;
          mbar_arrive_expect(xbar + b, kRowBytes);
          bulk_load(xb + b * kRowBytes, io.x + (size_t)row_of(k + 2) * kRowBytes, kRowBytes, xbar + b);
        }
      }
    }
    FP4AR_PHASE(6);   // encode pass 2 + push

    // ------------------------------------------------------------------ stage B: finish row k - lag_f
    if (fin) {
      const int row = frow;
      uint8_t* rec_own = recs + (kf % NREC) * kRecStride;
      if constexpr (!kTwoShot) {
        // ---- one-shot: every rank decodes every source in rank order ----
        float wrs[kPfSrc];
#pragma unroll
        for (int i = 0; i < NSG; i++) {
          const int s = window_source(i);
          wrs[i] = IN == 0 ? settle_rs(frs[i], fsrc[i], row, s, 1) : prm.gs[s];
        }
        float own_rs = 0.0f;
        if (IN == 0) own_rs = *reinterpret_cast<const float*>(rec_own + kQRowBytes);
        if (IN == 1) own_rs = prm.gs[me];
        auto fill = [&](int j, float* acc) {
          const int p = lane + 32 * (tw + T * j);
          uint4 wq[kPfSrc];
          uint32_t wsf[kPfSrc];
#pragma unroll
          for (int i = 0; i < NSG; i++) {
            if (kPfAll) { wq[i] = fq[j][i]; wsf[i] = fsf[j][i]; }
            else { wq[i] = poll_ld16(fsrc[i] + 16 * p); wsf[i] = poll_ld2(fsrc[i] + kValueBytes + 2 * p); }
          }
#pragma unroll
          for (int i = 0; i < NSG; i++)
            if (values_pending(wq[i]) | scales_pending(wsf[i])) poll_pair(fsrc[i], p, wq[i], wsf[i], row, window_source(i), 1);
          zero32(acc);
          if (!xport) {
#pragma unroll
            for (int i = 0; i <= NSG; i++) {
              if (IN != 2 && i == me) {
                const uint4 q = lds16(rec_own + 16 * p);
                const uint32_t sf2 = *reinterpret_cast<const uint16_t*>(rec_own + kValueBytes + 2 * p);
                decode_acc_lane(acc, q, sf2, own_rs, f);
              }
              if (i < NSG) decode_acc_lane(acc, wq[i], wsf[i], wrs[i], f);
            }
          }
        };
        auto extra = [&]() {
#pragma unroll
          for (int i = 0; i < NSG; i++) bulk_store(const_cast<char*>(fsrc[i]), sentinel, kRecPayload);
        };
        finish_row(row, fill, extra);
      } else {
        if (fin_owned) {
          // ---- two-shot, owned row: its re-encoding sits in the ring; every rank outputs the decode of that ----
          const float rs2 = *reinterpret_cast<const float*>(rec_own + kQRowBytes);
          auto fill = [&](int j, float* acc) {
            const int p = lane + 32 * (tw + T * j);
            zero32(acc);
            if (!xport) {
              const uint4 q = lds16(rec_own + 16 * p);
              const uint32_t sf2 = *reinterpret_cast<const uint16_t*>(rec_own + kValueBytes + 2 * p);
              decode_acc_lane(acc, q, sf2, rs2, f);
            }
          };
          auto extra = [&]() {};
          finish_row(row, fill, extra);
        } else {
          // ---- two-shot, row owned by a peer: its broadcast had lag_finish - lag_owner steps to arrive ----
          const char* src = fsrc[0];
          const int owner = row % P;
          const float rs = f_has_rs ? settle_rs(frs[0], src, row, owner, 3) : prm.gs[me];
          auto fill = [&](int j, float* acc) {
            const int p = lane + 32 * (tw + T * j);
            uint4 wq = fq[j][0];
            uint32_t wsf = fsf[j][0];
            if (values_pending(wq) | scales_pending(wsf)) poll_pair(src, p, wq, wsf, row, owner, 3);
            zero32(acc);
            if (!xport) decode_acc_lane(acc, wq, wsf, rs, f);
          };
          auto extra = [&]() { bulk_store(const_cast<char*>(src), sentinel, kRecPayload); };
          finish_row(row, fill, extra);
        }
      }
    }
    FP4AR_PHASE(7);   // finish
    if (leader) bulk_commit();
  }

  if (leader) bulk_wait_done<0>();
  __syncthreads();
  if (threadIdx.x == 0) io.ctrl[cta] = call + 1u;
}

}  // namespace fp4ar
