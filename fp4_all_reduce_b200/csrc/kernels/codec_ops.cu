// Stand-alone single-GPU kernels built from the same codec primitives as the fused AllReduce:
// row encode (dynamic row scale or static per-tensor scale), rank-ordered decode-sum, the two-shot
// owner step (decode-sum + re-encode + decode of the re-encoding), add + Gemma RMSNorm with BF16 /
// NVFP4 / MXFP8 output, and the sentinel fill of a receive window.
//
// All of them stream 12 KB rows: one warp per row, rows brought into shared memory by bulk
// asynchronous copies where the access pattern would otherwise be 64 B per lane, BF16 results staged
// in shared memory and written back with one bulk store per row.
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

// ---------------------------------------------------------------------------------------------
// encode: x [rows][6144] BF16 -> values / scales / row scales
// ---------------------------------------------------------------------------------------------
template <bool STATIC>
__global__ void __launch_bounds__(kOpsWarps * 32, 1)
encode_rows_kernel(const char* __restrict__ x, int rows, char* values, long vpitch, char* scales, long spitch,
                   float* row_scales, float inv_static, uint32_t* err) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WarpSmem ws = carve(smem, warp);
  if (lane == 0) { mbar_init(ws.bar, 1); mbar_init(ws.bar + 1, 1); }
  mbar_init_fence();
  __syncwarp();
  const int stride = gridDim.x * kOpsWarps;
  int row = blockIdx.x * kOpsWarps + warp;
  uint8_t* buf[2] = {ws.a, ws.b};
  if (lane == 0 && row < rows) { mbar_arrive_expect(ws.bar, kRowB); bulk_load(buf[0], x + (size_t)row * kRowB, kRowB, ws.bar); }
  for (int it = 0; row < rows; row += stride, it++) {
    const int nxt = row + stride;
    if (lane == 0 && nxt < rows) {
      mbar_arrive_expect(ws.bar + ((it + 1) & 1), kRowB);
      bulk_load(buf[(it + 1) & 1], x + (size_t)nxt * kRowB, kRowB, ws.bar + ((it + 1) & 1));
    }
    wait_row(ws.bar + (it & 1), (uint32_t)((it >> 1) & 1), err);
    char* vrow = values + (size_t)row * vpitch;
    char* srow = scales + (size_t)row * spitch;
    float rs;
    encode_row_from_smem(buf[it & 1], lane, inv_static, STATIC, rs,
                         [&](int p, uint4 q) { *reinterpret_cast<uint4*>(vrow + 16 * p) = q; },
                         [&](int p, uint32_t sf2) { *reinterpret_cast<uint16_t*>(srow + 2 * p) = (uint16_t)sf2; });
    if (!STATIC && lane == 0) row_scales[row] = rs;
    __syncwarp();   // every lane is done with buf[it & 1] before it is refilled two iterations later
  }
}

// ---------------------------------------------------------------------------------------------
// decode-sum: NS sources -> BF16 row; optional re-encode of the FP32 sum (two-shot owner step)
// ---------------------------------------------------------------------------------------------
struct SrcList {
  const char* base[kMaxRanksOps];
  const float* rs[kMaxRanksOps];
  float gs[kMaxRanksOps];
};

template <int NS, bool REENC>
__global__ void __launch_bounds__(kOpsWarps * 32, 1)
decode_sum_kernel(SrcList src, long pitch, int rows, char* rec_out, char* out) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int f = (lane >> 1) & 3;
  WarpSmem ws = carve(smem, warp);
  const int stride = gridDim.x * kOpsWarps;
  bool pending_store = false;
  for (int row = blockIdx.x * kOpsWarps + warp; row < rows; row += stride) {
    float rsv[NS];
#pragma unroll
    for (int s = 0; s < NS; s++) rsv[s] = src.rs[s] ? src.rs[s][row] : src.gs[s];
    auto sum_pair = [&](int p, float* acc) {
      zero32(acc);
#pragma unroll
      for (int s = 0; s < NS; s++) {
        const char* r = src.base[s] + (size_t)row * pitch;
        uint4 q = __ldcg(reinterpret_cast<const uint4*>(r + 16 * p));
        const uint32_t sf2 = __ldcg(reinterpret_cast<const unsigned short*>(r + kValueBytes + 2 * p));
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
    };
    if (lane == 0 && pending_store) bulk_wait_source_free<0>();
    __syncwarp();
    RowScale sc2;
    if (REENC) {
      float am = 0.0f;
#pragma unroll 1
      for (int j = 0; j < 6; j++) { float acc[32]; sum_pair(lane + 32 * j, acc); am = absmax32(acc, am); }
      sc2 = row_scale_from_amax(warp_max(am));
    }
#pragma unroll 1
    for (int j = 0; j < 6; j++) {
      const int p = lane + 32 * j;
      float acc[32];
      sum_pair(p, acc);
      if (REENC) {
        uint4 q;
        uint32_t sf2 = encode_pair_f32<true>(acc, sc2.inv, q);   // slot order in, slot order out
        // decode of the re-encoding, still in slot order
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
        perm4(q.x, q.y, q.z, q.w, f);
        if (f & 2) sf2 = ((sf2 & 0xffu) << 8) | (sf2 >> 8);
        char* r = rec_out + (size_t)row * kRecStride;
        *reinterpret_cast<uint4*>(r + 16 * p) = q;
        *reinterpret_cast<uint16_t*>(r + kValueBytes + 2 * p) = (uint16_t)sf2;
      }
      uint4 o[4];
      pack32_bf16(acc, o);
#pragma unroll
      for (int k = 0; k < 4; k++) sts16(ws.o + p * 64 + ((k ^ f) << 4), o[k]);
    }
    if (REENC && lane == 0) {
      const uint32_t b = __float_as_uint(sc2.rs);
      *reinterpret_cast<uint4*>(rec_out + (size_t)row * kRecStride + kQRowBytes) = make_uint4(b, b, b, b);
    }
    fence_smem_to_async();
    __syncwarp();
    if (lane == 0) { bulk_store(out + (size_t)row * kRowB, ws.o, kRowB); bulk_commit(); }
    pending_store = true;
  }
  if (lane == 0) bulk_wait_done<0>();
}

// ---------------------------------------------------------------------------------------------
// add + Gemma RMSNorm:  z = x + res, res_out = bf16(z), y = (bf16(z) * rinv) * (wbias + w)
// ---------------------------------------------------------------------------------------------
template <int EPI>
__global__ void __launch_bounds__(kOpsWarps * 32, 1)
add_rmsnorm_kernel(const char* __restrict__ x, const char* __restrict__ res_in, char* res_out,
                   const char* __restrict__ weight, float eps, float wbias, float qscale, char* out, char* outq,
                   int rows, uint32_t* err) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int f = (lane >> 1) & 3;
  WarpSmem ws = carve(smem, warp);
  if (lane == 0) { mbar_init(ws.bar, 1); }
  mbar_init_fence();
  __syncwarp();
  const int stride = gridDim.x * kOpsWarps;
  int it = 0;
  for (int row = blockIdx.x * kOpsWarps + warp; row < rows; row += stride, it++) {
    if (lane == 0) {
      bulk_wait_source_free<0>();     // the previous row's stores have left the buffers
      mbar_arrive_expect(ws.bar, 2 * kRowB);
      bulk_load(ws.a, x + (size_t)row * kRowB, kRowB, ws.bar);
      bulk_load(ws.b, res_in + (size_t)row * kRowB, kRowB, ws.bar);
    }
    wait_row(ws.bar, (uint32_t)(it & 1), err);
    uint4 zb[6][4];
    float g6[6];
#pragma unroll
    for (int j = 0; j < 6; j++) {
      const int p = lane + 32 * j;
      float acc[32];
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const uint4 c = lds16(ws.a + p * 64 + ((k ^ f) << 4));
        const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { const F2 t = bf16x2_to_f2(cw[i]); acc[8 * k + 2 * i] = t.lo; acc[8 * k + 2 * i + 1] = t.hi; }
        r[k] = lds16(ws.b + p * 64 + ((k ^ f) << 4));
      }
      const float sp = add_residual_sumsq(acc, r);
      pack32_bf16(acc, zb[j]);
#pragma unroll
      for (int k = 0; k < 4; k++) sts16(ws.b + p * 64 + ((k ^ f) << 4), zb[j][k]);
      g6[j] = warp_sum_butterfly(sp);
    }
    fence_smem_to_async();
    __syncwarp();
    if (lane == 0) bulk_store(res_out + (size_t)row * kRowB, ws.b, kRowB);
    float ss = g6[0];
#pragma unroll
    for (int g = 1; g < 6; g++) ss = __fadd_rn(ss, g6[g]);
    const float rinv = norm_rinv(ss, eps);
#pragma unroll
    for (int j = 0; j < 6; j++) {
      const int p = lane + 32 * j;
      uint4 wt[4];
#pragma unroll
      for (int k = 0; k < 4; k++) wt[k] = __ldg(reinterpret_cast<const uint4*>(weight + p * 64 + ((k ^ f) << 4)));
      float y[32];
      norm_pair(zb[j], wt, rinv, wbias, y);
      uint4 yb[4];
      pack32_bf16(y, yb);
      if (EPI == 1) {
#pragma unroll
        for (int k = 0; k < 4; k++) sts16(ws.o + p * 64 + ((k ^ f) << 4), yb[k]);
      } else if (EPI == 2) {
        uint4 q;
        uint32_t sf2 = quant_pair_nvfp4_out(yb, qscale, q);
        perm4(q.x, q.y, q.z, q.w, f);
        if (f & 2) sf2 = ((sf2 & 0xffu) << 8) | (sf2 >> 8);
        sts16(ws.o + p * 16, q);
        *reinterpret_cast<uint16_t*>(ws.o + kValueBytes + 2 * p) = (uint16_t)sf2;
      } else {
        uint4 v[2];
        const uint32_t e = quant_pair_mxfp8_out(yb, v);
        const uint32_t* vw = reinterpret_cast<const uint32_t*>(v);
#pragma unroll
        for (int k = 0; k < 4; k++)
          *reinterpret_cast<uint2*>(ws.o + p * 32 + ((k ^ f) << 3)) = make_uint2(vw[2 * k], vw[2 * k + 1]);
        ws.o[kHidden + p] = (uint8_t)e;
      }
    }
    fence_smem_to_async();
    __syncwarp();
    if (lane == 0) {
      if (EPI == 1) bulk_store(out + (size_t)row * kRowB, ws.o, kRowB);
      else if (EPI == 2) bulk_store(outq + (size_t)row * kQRowBytes, ws.o, kQRowBytes);
      else bulk_store(outq + (size_t)row * kMxRowBytes, ws.o, kMxRowBytes);
      bulk_commit();
    }
  }
  if (lane == 0) bulk_wait_done<0>();
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

// A word the kernels above set when a local row load did not arrive in time.
// One word per device for the whole process (allocated on the first use on that device, never freed).
static uint32_t* ops_error_word() {
  static std::mutex mu;
  static std::atomic<uint32_t*> p[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  uint32_t* w = p[dev].load(std::memory_order_acquire);
  if (w) return w;
  std::lock_guard<std::mutex> lock(mu);
  w = p[dev].load(std::memory_order_acquire);
  if (!w) {
    if (cudaMalloc(&w, 16) != cudaSuccess) return nullptr;
    cudaMemset(w, 0, 16);
    p[dev].store(w, std::memory_order_release);
  }
  return w;
}

static int ops_grid(int rows) {
  const int sms = device_sm_count();
  const int need = (rows + kOpsWarps - 1) / kOpsWarps;
  return need < sms ? (need > 0 ? need : 1) : sms;
}

// Raises a kernel's dynamic shared-memory limit once per (kernel, device); later calls are two atomic loads.
// (Every kernel of this file is launched with the one size kOpsSmem.)
struct SmemRaised {
  std::atomic<const void*> fn{nullptr};
  std::atomic<unsigned long long> devices{0};   // bit d: done on device d
};
static SmemRaised g_smem_raised[64];
template <class K>
static bool ensure_smem(K kernel, int bytes) {
  const void* key = reinterpret_cast<const void*>(kernel);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  SmemRaised* slot = nullptr;
  for (SmemRaised& e : g_smem_raised) {
    const void* cur = e.fn.load(std::memory_order_acquire);
    if (cur == nullptr) {
      const void* expected = nullptr;
      if (e.fn.compare_exchange_strong(expected, key, std::memory_order_acq_rel)) cur = key; else cur = expected;
    }
    if (cur == key) { slot = &e; break; }
  }
  if (slot && dev >= 0 && dev < 64 && ((slot->devices.load(std::memory_order_acquire) >> dev) & 1ull)) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  if (slot && dev >= 0 && dev < 64) slot->devices.fetch_or(1ull << dev, std::memory_order_release);
  return true;
}

}  // namespace fp4ar

using namespace fp4ar;

extern "C" int fp4ar_encode(const void* x, int rows, void* values, long vpitch, void* scales, long spitch,
                            float* row_scales, fp4ar_stream stream) {
  if (!x || !values || !scales || !row_scales || rows < 0 || vpitch < kValueBytes || spitch < kScaleBytes) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)x | (uintptr_t)values | (uintptr_t)vpitch) & 15) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)scales | (uintptr_t)spitch) & 1) return FP4AR_ERR_ARGUMENT;
  if (rows == 0) return FP4AR_OK;
  uint32_t* err = ops_error_word();
  if (!err || !ensure_smem(encode_rows_kernel<false>, kOpsSmem)) return cuda_fail();
  encode_rows_kernel<false><<<ops_grid(rows), kOpsWarps * 32, kOpsSmem, (cudaStream_t)stream>>>(
      (const char*)x, rows, (char*)values, vpitch, (char*)scales, spitch, row_scales, 0.0f, err);
  return cuda_check_launch();
}

extern "C" int fp4ar_encode_static(const void* x, int rows, float gs, void* qrows, fp4ar_stream stream) {
  if (!x || !qrows || rows < 0 || !(gs > 0.0f)) return FP4AR_ERR_ARGUMENT;
  if (((uintptr_t)x | (uintptr_t)qrows) & 15) return FP4AR_ERR_ARGUMENT;
  if (rows == 0) return FP4AR_OK;
  uint32_t* err = ops_error_word();
  if (!err || !ensure_smem(encode_rows_kernel<true>, kOpsSmem)) return cuda_fail();
  encode_rows_kernel<true><<<ops_grid(rows), kOpsWarps * 32, kOpsSmem, (cudaStream_t)stream>>>(
      (const char*)x, rows, (char*)qrows, kQRowBytes, (char*)qrows + kValueBytes, kQRowBytes, nullptr, 1.0f / gs, err);
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
  const int grid = ops_grid(rows), blk = kOpsWarps * 32;
#define FP4AR_DEC_CASE(N)                                                                                   \
  case N:                                                                                                   \
    if (!ensure_smem(decode_sum_kernel<N, REENC>, kOpsSmem)) return cuda_fail();                             \
    decode_sum_kernel<N, REENC><<<grid, blk, kOpsSmem, st>>>(sl, pitch, rows, (char*)rec_out, (char*)out);  \
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
  uint32_t* err = ops_error_word();
  if (!err) return cuda_fail();
  const int grid = ops_grid(rows), blk = kOpsWarps * 32;
  cudaStream_t st = (cudaStream_t)stream;
#define FP4AR_NORM_CASE(E)                                                                                         \
  case E:                                                                                                          \
    if (!ensure_smem(add_rmsnorm_kernel<E>, kOpsSmem)) return cuda_fail();                                          \
    add_rmsnorm_kernel<E><<<grid, blk, kOpsSmem, st>>>((const char*)x, (const char*)res_in, (char*)res_out,        \
                                                       (const char*)weight, eps, wbias, qscale, (char*)out,        \
                                                       (char*)outq, rows, err);                                    \
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
