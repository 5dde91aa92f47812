// Warp-per-row building blocks shared by the stand-alone codec kernels and the comparison variants:
// per-warp shared-memory carving, a bounded wait on a row load, and the row encoder that reads a BF16 row from
// shared memory and hands out canonical 16-byte value groups and 2-byte scale pairs.
#pragma once
#include "../include/fp4ar_codec.cuh"
#include "../include/fp4ar_async.cuh"

namespace fp4ar {

constexpr int kRowB = kHidden * 2;
constexpr int kOpsWarps = 6;     // warps per CTA; each owns 36 KB of shared memory

__device__ __forceinline__ void perm4(uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d, int f) {
  if (f & 1) { uint32_t t = a; a = b; b = t; t = c; c = d; d = t; }
  if (f & 2) { uint32_t t = a; a = c; c = t; t = b; b = d; d = t; }
}

// Bounded wait on a row load; a failure only flags the error word (the op's output is then undefined).
__device__ __forceinline__ void wait_row(uint64_t* bar, uint32_t parity, uint32_t* err) {
  if (mbar_test(bar, parity)) return;
  const unsigned long long t0 = global_timer_ns();
  uint32_t n = 0;
  while (!mbar_test(bar, parity)) {
    if ((++n & 63u) == 0u && global_timer_ns() - t0 > 2000000000ull) { atomicExch(err, 1u); return; }
  }
}

struct WarpSmem {
  uint8_t* a;      // 12 KB row buffer
  uint8_t* b;      // 12 KB row buffer
  uint8_t* o;      // 12 KB output staging
  uint64_t* bar;   // 2 mbarriers
};
__device__ __forceinline__ WarpSmem carve(uint8_t* smem, int warp) {
  WarpSmem w;
  uint8_t* base = smem + (size_t)warp * (3 * kRowB + 64);
  w.a = base; w.b = base + kRowB; w.o = base + 2 * kRowB;
  w.bar = reinterpret_cast<uint64_t*>(base + 3 * kRowB);
  return w;
}
constexpr int kOpsSmem = kOpsWarps * (3 * kRowB + 64);

// Encode the BF16 row sitting in shared memory at `xrow`; lane l handles pairs l + 32 j.
// Writes canonical 16 B value groups and 2 B scale pairs through the two callbacks.
template <class PutQ, class PutS>
__device__ __forceinline__ void encode_row_from_smem(const uint8_t* xrow, int lane, float inv_fixed, bool use_fixed,
                                                     float& rs_out, PutQ put_q, PutS put_s) {
  const int f = (lane >> 1) & 3;
  uint32_t bmp[6];
  float am = 0.0f;
#pragma unroll
  for (int j = 0; j < 6; j++) {
    const int p = lane + 32 * j;
    const __nv_bfloat162 z2 = __floats2bfloat162_rn(0.0f, 0.0f);
    __nv_bfloat162 ma = z2, mb = z2;
    ma = chunk_absmax(lds16(xrow + p * 64 + ((0 ^ f) << 4)), ma);
    ma = chunk_absmax(lds16(xrow + p * 64 + ((1 ^ f) << 4)), ma);
    mb = chunk_absmax(lds16(xrow + p * 64 + ((2 ^ f) << 4)), mb);
    mb = chunk_absmax(lds16(xrow + p * 64 + ((3 ^ f) << 4)), mb);
    const uint32_t xa = bf16x2_hmax_bits(ma), xb = bf16x2_hmax_bits(mb);
    bmp[j] = (f & 2) ? (xb | (xa << 16)) : (xa | (xb << 16));
    am = fmaxf(am, __uint_as_float(max(xa, xb) << 16));
  }
  am = warp_max(am);
  const RowScale sc = row_scale_from_amax(am);
  const float inv = use_fixed ? inv_fixed : sc.inv;
  rs_out = sc.rs;
#pragma unroll
  for (int j = 0; j < 6; j++) {
    const int p = lane + 32 * j;
    const float bm0 = __uint_as_float(bmp[j] << 16), bm1 = __uint_as_float(bmp[j] & 0xffff0000u);
    float m0, m1;
    const uint32_t sf2 = pair_block_scales(bm0, bm1, inv, m0, m1);
    const float mlo = (f & 2) ? m1 : m0, mhi = (f & 2) ? m0 : m1;
    uint32_t w0 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((0 ^ f) << 4)), mlo);
    uint32_t w1 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((1 ^ f) << 4)), mlo);
    uint32_t w2 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((2 ^ f) << 4)), mhi);
    uint32_t w3 = quant_chunk_bf16<true>(lds16(xrow + p * 64 + ((3 ^ f) << 4)), mhi);
    perm4(w0, w1, w2, w3, f);
    put_q(p, make_uint4(w0, w1, w2, w3));
    put_s(p, sf2);
  }
}

}  // namespace fp4ar
