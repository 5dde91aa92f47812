// Stand-alone single-GPU kernels built from the same codec primitives as the fused AllReduce:
// row encode (dynamic row scale or static per-tensor scale), rank-ordered decode-sum, the two-shot
// owner step (decode-sum + re-encode + decode of the re-encoding), add + Gemma RMSNorm with BF16 /
// NVFP4 / MXFP8 output, and the sentinel fill of a receive window.
//
// All of them stream 12 KB rows through teams of 192 threads (one pair of a row per thread, several teams per
// SM); see "Row teams" below.
//
// Reference project counterparts: bench/codec/codec_bench.cu:139-590 (k_enc_*, k_dec_*, k_ts_*),
// kernels/push/tp2_l2.cu:967-978 (fill_sentinel), bench/fused_norm/drv_norm.cu:75-123 (ref_norm).
#include <atomic>
#include <mutex>
#include "../include/fp4ar.h"
#include "../include/fp4ar_codec.cuh"
#include "../include/fp4ar_async.cuh"
#include "host_util.h"
#include "row_ops.cuh"

namespace fp4ar {

// =============================================================================================
// Row teams.  Every kernel below gives a row to a team of 192 threads (6 warps): thread t owns pair t of the
// row (values 32t .. 32t+31: 64 B of BF16, 16 B of E2M1, 2 scale bytes), so the compact NVFP4 fields are read
// and written fully coalesced straight from registers.  The 64-byte BF16 pieces go through a 2 KB staging area
// per warp: global memory is touched with consecutive 16-byte chunks per lane (512 B per warp instruction) and
// the area is transposed into "own pair" order through a bank-conflict-free swizzle.  A CTA is one team; several
// CTAs share an SM (the kernels need no more than 12.5 KB of shared memory and 64-112 registers), so the loads of
// one team overlap the arithmetic of the others.  Teams walk rows with a grid stride and take U rows per trip,
// issuing every load of the trip before the first use.
// =============================================================================================
constexpr int kTeamThreads = kPairs;          // 192
constexpr int kTeamWarps = kTeamThreads / 32;  // 6
constexpr int kStageBytes = 2048;              // per warp: 32 pairs x 64 B

// chunk k (16 B) of lane l's pair inside the warp's staging area
__device__ __forceinline__ int stage_off(int l, int k) { return l * 64 + ((k ^ ((l >> 1) & 3)) << 4); }

// Global -> registers: the warp's 32 pairs (2 KB at `unit`) as four 16-byte chunks per lane, in chunk order.
// load_issue() starts the coalesced loads; stage_in() transposes them through the staging area.
__device__ __forceinline__ void load_issue(const char* unit, int lane, uint4* raw) {
#pragma unroll
  for (int it = 0; it < 4; it++) raw[it] = __ldcs(reinterpret_cast<const uint4*>(unit + (it * 32 + lane) * 16));
}
__device__ __forceinline__ void stage_in(uint8_t* stage, int lane, const uint4* raw, uint4* mine) {
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 4; it++) {
    const int c = it * 32 + lane;
    sts16(stage + stage_off(c >> 2, c & 3), raw[it]);
  }
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 4; k++) mine[k] = lds16(stage + stage_off(lane, k));
}
// Registers -> global: the reverse path.
__device__ __forceinline__ void stage_out(uint8_t* stage, int lane, const uint4* mine, char* unit) {
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 4; k++) sts16(stage + stage_off(lane, k), mine[k]);
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 4; it++) {
    const int c = it * 32 + lane;
    __stcs(reinterpret_cast<uint4*>(unit + c * 16), lds16(stage + stage_off(c >> 2, c & 3)));
  }
}

// One float per warp -> the same six floats in every thread of the team (slot = parity of the exchange).
__device__ __forceinline__ void team_exchange6(float* xchg, int& phase, int warp, int lane, float mine, float* all6) {
  float* slot = xchg + 8 * (phase & 1);
  phase++;
  if (lane == 0) slot[warp] = mine;
  __syncthreads();
#pragma unroll
  for (int g = 0; g < kTeamWarps; g++) all6[g] = slot[g];
}

// acc (natural order) += decode of one pair of one source
__device__ __forceinline__ void decode_acc_natural(float* acc, uint4 q, uint32_t sf2, float rs) {
  const F2 e = e4m3_unpack2(sf2);
  const F2 sa = f2_splat(__fmul_rn(e.lo, rs)), sb = f2_splat(__fmul_rn(e.hi, rs));
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

// ---------------------------------------------------------------------------------------------
// encode: x [rows][6144] BF16 -> values / scales / row scales
// ---------------------------------------------------------------------------------------------
template <bool STATIC>
__global__ void __launch_bounds__(kTeamThreads, 4)
encode_rows_kernel(const char* __restrict__ x, int rows, char* values, long vpitch, char* scales, long spitch,
                   float* row_scales, float inv_static) {
  __shared__ __align__(128) uint8_t stage_all[kTeamWarps * kStageBytes];
  __shared__ float xchg[16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, p = threadIdx.x;
  uint8_t* stage = stage_all + warp * kStageBytes;
  int phase = 0;
  constexpr int U = 2;
  for (int row0 = blockIdx.x * U; row0 < rows; row0 += gridDim.x * U) {
    uint4 raw[U][4];
#pragma unroll
    for (int u = 0; u < U; u++)
      if (row0 + u < rows) load_issue(x + (size_t)(row0 + u) * kRowB + warp * kStageBytes, lane, raw[u]);
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int row = row0 + u;
      if (row >= rows) break;           // uniform over the team
      uint4 c[4];
      stage_in(stage, lane, raw[u], c);
      const __nv_bfloat162 z2 = __floats2bfloat162_rn(0.0f, 0.0f);
      const uint32_t xa = bf16x2_hmax_bits(chunk_absmax(c[1], chunk_absmax(c[0], z2)));
      const uint32_t xb = bf16x2_hmax_bits(chunk_absmax(c[3], chunk_absmax(c[2], z2)));
      const float bm0 = __uint_as_float(xa << 16), bm1 = __uint_as_float(xb << 16);
      float inv = inv_static, rs = 0.0f;
      if (!STATIC) {
        float g6[kTeamWarps];
        team_exchange6(xchg, phase, warp, lane, warp_max(fmaxf(bm0, bm1)), g6);
        float am = g6[0];
#pragma unroll
        for (int g = 1; g < kTeamWarps; g++) am = fmaxf(am, g6[g]);
        const RowScale sc = row_scale_from_amax(am);
        inv = sc.inv; rs = sc.rs;
      }
      float m0, m1;
      const uint32_t sf2 = pair_block_scales(bm0, bm1, inv, m0, m1);
      uint4 q;
      q.x = quant_chunk_bf16<true>(c[0], m0); q.y = quant_chunk_bf16<true>(c[1], m0);
      q.z = quant_chunk_bf16<true>(c[2], m1); q.w = quant_chunk_bf16<true>(c[3], m1);
      __stcs(reinterpret_cast<uint4*>(values + (size_t)row * vpitch + 16 * p), q);
      *reinterpret_cast<uint16_t*>(scales + (size_t)row * spitch + 2 * p) = (uint16_t)sf2;
      if (!STATIC && p == 0) row_scales[row] = rs;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// decode-sum: NS sources -> BF16 row; optional re-encode of the FP32 sum (two-shot owner step): the sum is
// decoded ONCE, kept in registers across the row-maximum exchange, re-encoded, and the re-encoding decoded.
// ---------------------------------------------------------------------------------------------
struct SrcList {
  const char* base[kMaxRanksOps];
  const float* rs[kMaxRanksOps];
  float gs[kMaxRanksOps];
};

// Rows whose loads a team issues together before the first use (bytes in flight against registers).
__host__ __device__ constexpr int decode_rows_per_trip(int ns, bool reenc) {
  return reenc ? 1 : (ns == 1 ? 4 : (ns == 2 ? 2 : 1));
}
// Four teams per SM (24 warps, at most 80 registers) for every shape: these kernels are bound by instruction issue
// (about three instructions per decoded value), so warps to choose from count for more than loads in flight per
// thread.  Measured at 16384 rows: eight sources 143 us at three teams / 90 registers, 122 us at four / 78; the
// owner step 128 us at three teams with two rows per trip, 122 us at four with one.
constexpr int kDecodeTeamsPerSm = 4;

template <int NS, bool REENC>
__global__ void __launch_bounds__(kTeamThreads, kDecodeTeamsPerSm)
decode_sum_kernel(SrcList src, long pitch, int rows, char* rec_out, char* out) {
  __shared__ __align__(128) uint8_t stage_all[kTeamWarps * kStageBytes];
  __shared__ float xchg[16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, p = threadIdx.x;
  uint8_t* stage = stage_all + warp * kStageBytes;
  int phase = 0;
  constexpr int U = decode_rows_per_trip(NS, REENC);
  for (int row0 = blockIdx.x * U; row0 < rows; row0 += gridDim.x * U) {
    uint4 q[U][NS];
    uint32_t sf[U][NS];
    float rsv[U][NS];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int row = row0 + u < rows ? row0 + u : rows - 1;     // clamped: the extra loads are discarded
#pragma unroll
      for (int s = 0; s < NS; s++) {
        const char* r = src.base[s] + (size_t)row * pitch;
        q[u][s] = __ldcs(reinterpret_cast<const uint4*>(r + 16 * p));
        sf[u][s] = __ldcs(reinterpret_cast<const unsigned short*>(r + kValueBytes + 2 * p));
        rsv[u][s] = src.rs[s] ? __ldg(src.rs[s] + row) : src.gs[s];
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int row = row0 + u;
      if (row >= rows) break;           // uniform over the team
      float acc[32];
      zero32(acc);
#pragma unroll
      for (int s = 0; s < NS; s++) decode_acc_natural(acc, q[u][s], sf[u][s], rsv[u][s]);
      if (REENC) {
        float g6[kTeamWarps];
        const float bm0 = absmax16(acc), bm1 = absmax16(acc + 16);
        team_exchange6(xchg, phase, warp, lane, warp_max(fmaxf(bm0, bm1)), g6);
        float am = g6[0];
#pragma unroll
        for (int g = 1; g < kTeamWarps; g++) am = fmaxf(am, g6[g]);
        const RowScale sc2 = row_scale_from_amax(am);
        uint4 qq;
        const uint32_t sf2 = encode_pair_f32<true>(acc, bm0, bm1, [&](float b0, float b1, float& m0, float& m1) {
          return pair_block_scales(b0, b1, sc2.inv, m0, m1);
        }, qq);
        char* r = rec_out + (size_t)row * kRecStride;
        *reinterpret_cast<uint4*>(r + 16 * p) = qq;
        *reinterpret_cast<uint16_t*>(r + kValueBytes + 2 * p) = (uint16_t)sf2;
        if (p == 0) {
          const uint32_t b = __float_as_uint(sc2.rs);
          *reinterpret_cast<uint4*>(r + kQRowBytes) = make_uint4(b, b, b, b);
        }
        zero32(acc);
        decode_acc_natural(acc, qq, sf2, sc2.rs);       // every rank outputs the decode of the re-encoding
      }
      uint4 o[4];
      pack32_bf16(acc, o);
      stage_out(stage, lane, o, out + (size_t)row * kRowB + warp * kStageBytes);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// add + Gemma RMSNorm:  z = x + res, res_out = bf16(z), y = (bf16(z) * rinv) * (wbias + w)
// The sum of squares follows the fixed tree of the host model: per pair (t0 + t1) + (t2 + t3) over its four
// chunk sums, a butterfly over the 32 pairs of a group (= one warp here), then the six groups in order.
// ---------------------------------------------------------------------------------------------
template <int EPI>
__global__ void __launch_bounds__(kTeamThreads, 3)
add_rmsnorm_kernel(const char* __restrict__ x, const char* __restrict__ res_in, char* res_out,
                   const char* __restrict__ weight, float eps, float wbias, float qscale, char* out, char* outq,
                   int rows) {
  __shared__ __align__(128) uint8_t stage_all[kTeamWarps * kStageBytes];
  __shared__ float xchg[16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, p = threadIdx.x;
  uint8_t* stage = stage_all + warp * kStageBytes;
  int phase = 0;
  // this thread's 32 weights never change: fetched once
  uint4 wt[4];
  {
    uint4 raw[4];
    load_issue(weight + warp * kStageBytes, lane, raw);
    stage_in(stage, lane, raw, wt);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 rx[4], rr[4];
    load_issue(x + (size_t)row * kRowB + warp * kStageBytes, lane, rx);
    load_issue(res_in + (size_t)row * kRowB + warp * kStageBytes, lane, rr);
    uint4 cx[4], cr[4];
    stage_in(stage, lane, rx, cx);
    stage_in(stage, lane, rr, cr);
    float acc[32];
    {
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(cx);
#pragma unroll
      for (int i = 0; i < 16; i++) { const F2 t = bf16x2_to_f2(xw[i]); acc[2 * i] = t.lo; acc[2 * i + 1] = t.hi; }
    }
    const float sp = add_residual_sumsq(acc, cr);
    uint4 zb[4];
    pack32_bf16(acc, zb);
    stage_out(stage, lane, zb, res_out + (size_t)row * kRowB + warp * kStageBytes);
    float g6[kTeamWarps];
    team_exchange6(xchg, phase, warp, lane, warp_sum_butterfly(sp), g6);
    float ss = g6[0];
#pragma unroll
    for (int g = 1; g < kTeamWarps; g++) ss = __fadd_rn(ss, g6[g]);
    const float rinv = norm_rinv(ss, eps);
    float y[32];
    norm_pair(zb, wt, rinv, wbias, y);
    uint4 yb[4];
    pack32_bf16(y, yb);
    if (EPI == 1) {
      stage_out(stage, lane, yb, out + (size_t)row * kRowB + warp * kStageBytes);
    } else if (EPI == 2) {
      uint4 q;
      const uint32_t sf2 = quant_pair_nvfp4_out(yb, qscale, q);
      char* r = outq + (size_t)row * kQRowBytes;
      __stcs(reinterpret_cast<uint4*>(r + 16 * p), q);
      *reinterpret_cast<uint16_t*>(r + kValueBytes + 2 * p) = (uint16_t)sf2;
    } else {
      uint4 v[2];
      const uint32_t e = quant_pair_mxfp8_out(yb, v);
      char* r = outq + (size_t)row * kMxRowBytes;
      __stcs(reinterpret_cast<uint4*>(r + 32 * p), v[0]);
      __stcs(reinterpret_cast<uint4*>(r + 32 * p + 16), v[1]);
      r[kHidden + p] = (char)(uint8_t)e;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// sentinel fill of a window made of `nbuf` buffers of `buf_bytes` (slots of kRecStride from each buffer start)
// ---------------------------------------------------------------------------------------------
__global__ void fill_sentinel_kernel(uint4* win, size_t buf_units, int nbuf) {
  const size_t total = buf_units * nbuf;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t u = (i % buf_units) % (kRecStride / 16);
    uint4 v;
    if (u < kValueBytes / 16) v = make_uint4(kSentWord, kSentWord, kSentWord, kSentWord);
    else if (u < kQRowBytes / 16) v = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
    else if (u == kQRowBytes / 16) v = make_uint4(kSentRow, kSentRow, kSentRow, kSentRow);
    else v = make_uint4(0, 0, 0, 0);
    win[i] = v;
  }
}

// Persistent grid of row teams: enough CTAs to fill every SM `per_sm` times, never more than there are trips.
static int team_grid(int rows, int rows_per_trip, int per_sm) {
  const int trips = (rows + rows_per_trip - 1) / rows_per_trip;
  const int cap = device_sm_count() * per_sm;
  return trips < cap ? (trips > 0 ? trips : 1) : cap;
}

}  // namespace fp4ar

using namespace fp4ar;

extern "C" int fp4ar_encode(const void* x, int rows, void* values, long vpitch, void* scales, long spitch,
                            float* row_scales, fp4ar_stream stream) {
  if (!x || !values || !scales || !row_scales || rows < 0 || vpitch < kValueBytes || spitch < kScaleBytes) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)x | (uintptr_t)values | (uintptr_t)vpitch) & 15) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)scales | (uintptr_t)spitch) & 1) return FP4AR_ERR_ARGUMENT;
  if (rows == 0) return FP4AR_OK;
  encode_rows_kernel<false><<<team_grid(rows, 2, 4), kTeamThreads, 0, (cudaStream_t)stream>>>(
      (const char*)x, rows, (char*)values, vpitch, (char*)scales, spitch, row_scales, 0.0f);
  return cuda_check_launch();
}

extern "C" int fp4ar_encode_static(const void* x, int rows, float gs, void* qrows, fp4ar_stream stream) {
  if (!x || !qrows || rows < 0 || !(gs > 0.0f)) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)x | (uintptr_t)qrows) & 15) return FP4AR_ERR_ARGUMENT;
  if (rows == 0) return FP4AR_OK;
  encode_rows_kernel<true><<<team_grid(rows, 2, 4), kTeamThreads, 0, (cudaStream_t)stream>>>(
      (const char*)x, rows, (char*)qrows, kQRowBytes, (char*)qrows + kValueBytes, kQRowBytes, nullptr, 1.0f / gs);
  return cuda_check_launch();
}

template <bool REENC>
static int launch_decode(int nsrc, const void* const* src, long pitch, const float* const* rs, const float* gs, int rows,
                         void* rec_out, void* out, cudaStream_t st) {
  if (nsrc < 1 || nsrc > FP4AR_MAX_RANKS || !src || !out || rows < 0 || pitch < kQRowBytes || (pitch & 15)) return FP4AR_ERR_ARGUMENT;
  if (REENC && !rec_out) return FP4AR_ERR_ARGUMENT;
  SrcList sl;
  for (int s = 0; s < kMaxRanksOps; s++) { sl.base[s] = nullptr; sl.rs[s] = nullptr; sl.gs[s] = 0.0f; }
  for (int s = 0; s < nsrc; s++) {
    if (!src[s] || ((uintptr_t)src[s] & 15)) return FP4AR_ERR_ARGUMENT;
    sl.base[s] = (const char*)src[s];
    sl.rs[s] = rs ? rs[s] : nullptr;
    if (!sl.rs[s]) { if (!gs) return FP4AR_ERR_ARGUMENT; sl.gs[s] = gs[s]; }
  }
  if (rows == 0) return FP4AR_OK;
  const int grid = team_grid(rows, decode_rows_per_trip(nsrc, REENC), kDecodeTeamsPerSm);
#define FP4AR_DEC_CASE(N)                                                                                          \
  case N:                                                                                                          \
    decode_sum_kernel<N, REENC><<<grid, kTeamThreads, 0, st>>>(sl, pitch, rows, (char*)rec_out, (char*)out);       \
    break;
  switch (nsrc) {
    FP4AR_DEC_CASE(1) FP4AR_DEC_CASE(2) FP4AR_DEC_CASE(3) FP4AR_DEC_CASE(4)
    FP4AR_DEC_CASE(5) FP4AR_DEC_CASE(6) FP4AR_DEC_CASE(7) FP4AR_DEC_CASE(8)
  }
#undef FP4AR_DEC_CASE
  return cuda_check_launch();
}

extern "C" int fp4ar_decode_sum(int nsrc, const void* const* src, long pitch, const float* const* rs, const float* gs,
                                int rows, void* out, fp4ar_stream stream) {
  return launch_decode<false>(nsrc, src, pitch, rs, gs, rows, nullptr, out, (cudaStream_t)stream);
}
extern "C" int fp4ar_reduce_reencode(int nsrc, const void* const* src, long pitch, const float* const* rs,
                                     const float* gs, int rows, void* rec_out, void* out, fp4ar_stream stream) {
  return launch_decode<true>(nsrc, src, pitch, rs, gs, rows, rec_out, out, (cudaStream_t)stream);
}

extern "C" int fp4ar_add_rmsnorm(const void* x, const void* res_in, void* res_out, const void* weight, float eps,
                                 float wbias, int epilogue, float qscale, void* out, void* outq, int rows,
                                 fp4ar_stream stream) {
  if (!x || !res_in || !res_out || !weight || rows < 0) return FP4AR_ERR_ARGUMENT;
  if (epilogue < 1 || epilogue > 3) return FP4AR_ERR_ARGUMENT;
  if (epilogue == 1 ? !out : !outq) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)x | (uintptr_t)res_in | (uintptr_t)res_out | (uintptr_t)weight | (uintptr_t)out | (uintptr_t)outq) & 15)
    return FP4AR_ERR_ARGUMENT;
  if (rows == 0) return FP4AR_OK;
  const int grid = team_grid(rows, 1, 3);
  cudaStream_t st = (cudaStream_t)stream;
#define FP4AR_NORM_CASE(E)                                                                                         \
  case E:                                                                                                          \
    add_rmsnorm_kernel<E><<<grid, kTeamThreads, 0, st>>>((const char*)x, (const char*)res_in, (char*)res_out,      \
                                                         (const char*)weight, eps, wbias, qscale, (char*)out,      \
                                                         (char*)outq, rows);                                       \
    break;
  switch (epilogue) { FP4AR_NORM_CASE(1) FP4AR_NORM_CASE(2) FP4AR_NORM_CASE(3) }
#undef FP4AR_NORM_CASE
  return cuda_check_launch();
}

extern "C" int fp4ar_fill_sentinel(void* window, size_t buffer_bytes, int nbuffers, fp4ar_stream stream) {
  if (!window || ((uintptr_t)window & 15) || (buffer_bytes & 15) || nbuffers < 1) return FP4AR_ERR_ARGUMENT;
  fill_sentinel_kernel<<<1024, 256, 0, (cudaStream_t)stream>>>((uint4*)window, buffer_bytes / 16, nbuffers);
  return cuda_check_launch();
}

// ---------------------------------------------------------------------------------------------
// Self-test of the division-free multiplier: for one biased exponent of inv, every mantissa and every positive
// finite E4M3 byte, count the cases where it differs from the IEEE quotient (must be zero).
// Reference project counterpart: test T2 of bench/codec/codec_bench.cu:45-64.
// ---------------------------------------------------------------------------------------------
namespace fp4ar {
__global__ void scale_division_selftest_kernel(uint32_t exp_biased, unsigned long long* mismatches) {
  __shared__ float2 tab[128];
  fill_scale_lut(tab, threadIdx.x, blockDim.x);
  __syncthreads();
  unsigned long long bad = 0;
  for (uint32_t man = blockIdx.x * blockDim.x + threadIdx.x; man < (1u << 23); man += gridDim.x * blockDim.x) {
    const float inv = __uint_as_float((exp_biased << 23) | man);
    for (int b = 1; b < 127; b++) {
      const float want = __fdiv_rn(inv, tab[b].x);
      const float got = lut_multiplier(inv, tab[b], true);
      bad += __float_as_uint(want) != __float_as_uint(got);
    }
  }
  if (bad) atomicAdd(mismatches, bad);
}
}  // namespace fp4ar

extern "C" int fp4ar_selftest_scale_division(int exp_biased, unsigned long long* device_mismatch_counter, fp4ar_stream stream) {
  if (exp_biased < 27 || exp_biased > 227 || !device_mismatch_counter) return FP4AR_ERR_ARGUMENT;   // 2^-100 .. 2^100
  fp4ar::scale_division_selftest_kernel<<<1184, 256, 0, (cudaStream_t)stream>>>((uint32_t)exp_biased, device_mismatch_counter);
  return fp4ar::cuda_check_launch();
}

// ---------------------------------------------------------------------------------------------
// fp4ar_reduce_reencode_noalloc (declared and documented in include/fp4ar_noalloc.h): the owner step with
// its record buffer in a fixed device array instead of caller memory.  No counterpart in the reference.
// ---------------------------------------------------------------------------------------------
#include "../include/fp4ar_noalloc.h"
#include <cstdio>
#include <mutex>

// The records of one call: FP4AR_NOALLOC_MAX_ROWS slots of kRecStride bytes.  In host code this name is only a
// handle for cudaGetSymbolAddress; the kernel receives the device address looked up below.
static __device__ __align__(256) unsigned char g_noalloc_records[(size_t)FP4AR_NOALLOC_MAX_ROWS * fp4ar::kRecStride];

static thread_local char g_noalloc_error[256] = "";

static int noalloc_fail(int code, const char* text) {
  std::snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s", text);
  return code;
}

// Device address of the array on the current device; looked up once per device, with that device current.
// After the first call on a device this is one atomic load: no lock, no CUDA call besides cudaGetDevice.
static void* noalloc_records_on_current_device() {
  static std::mutex mu;
  static std::atomic<void*> addr[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  void* p = addr[dev].load(std::memory_order_acquire);
  if (p) return p;
  std::lock_guard<std::mutex> lock(mu);
  p = addr[dev].load(std::memory_order_acquire);
  if (!p) {
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_records);
    if (e != cudaSuccess || !p) {
      fp4ar::set_last_cuda_error(e, "cudaGetSymbolAddress(g_noalloc_records)");
      return nullptr;
    }
    addr[dev].store(p, std::memory_order_release);
  }
  return p;
}

extern "C" const char* fp4ar_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int fp4ar_reduce_reencode_noalloc(int nsrc, const void* const* src, long pitch, const float* const* rs,
                                             const float* gs, int rows, void* out_bf16, fp4ar_stream stream) {
  g_noalloc_error[0] = 0;
  if (rows > FP4AR_NOALLOC_MAX_ROWS) {
    char msg[200];
    std::snprintf(msg, sizeof(msg), "fp4ar_reduce_reencode_noalloc: %d rows exceed the built-in record array of %d rows",
                  rows, FP4AR_NOALLOC_MAX_ROWS);
    return noalloc_fail(FP4AR_ERR_ARGUMENT, msg);
  }
  void* records = noalloc_records_on_current_device();
  if (!records)
    return noalloc_fail(FP4AR_ERR_CUDA, "fp4ar_reduce_reencode_noalloc: the record array's device address is unavailable");
  const int rc = launch_decode<true>(nsrc, src, pitch, rs, gs, rows, records, out_bf16, (cudaStream_t)stream);
  if (rc == FP4AR_ERR_ARGUMENT) return noalloc_fail(rc, "fp4ar_reduce_reencode_noalloc: bad source list, pitch or output pointer");
  if (rc != FP4AR_OK) return noalloc_fail(rc, "fp4ar_reduce_reencode_noalloc: the launch failed (see fp4ar_last_cuda_error)");
  return FP4AR_OK;
}
