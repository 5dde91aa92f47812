// Device side of the NVFP4 row transport for sm_100a: scalar / packed conversion primitives, the
// block encoder, the decode-accumulate step and the Gemma RMSNorm epilogue math.
//
// Wire format of one 6144-wide row (bit-exact with the reference project's "codec spec v2",
// include/fp4_codec.cuh:14-25,82-133 there):
//   values   3072 B  E2M1, element 2i in the low nibble of byte i, -0 (0x8) canonicalised to +0
//   scales    384 B  E4M3 (satfinite), scale k covers elements 16k..16k+15
//   rowscale    4 B  FP32 rs = amax/2688 (absent when the producer used a static per-rank scale)
// Sentinels that no encoder can emit mark "not yet written" memory: value word 0x88888888,
// scale byte 0xFF, row scale -0.0f.
//
// Every arithmetic step is an IEEE round-to-nearest operation so that the host model
// (csrc/oracle/oracle.cpp) reproduces it bit for bit.  Compile with
//   -gencode arch=compute_100a,code=sm_100a   (the e2m1 conversions need the arch-specific target)
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace fp4ar {

constexpr int kHidden = 6144;
constexpr int kPairs = kHidden / 32;          // 192 pairs of two 16-value blocks
constexpr int kValueBytes = kHidden / 2;      // 3072
constexpr int kScaleBytes = kHidden / 16;     // 384
constexpr int kQRowBytes = kValueBytes + kScaleBytes;  // 3456: NVFP4 row without row scale
constexpr int kRecPayload = kQRowBytes + 16;  // 3472: + FP32 row scale replicated 4x (16 B granule)
constexpr int kRecStride = 3584;              // receive-slot pitch: 14 x 256 B so slots start on NVLink packet boundaries
constexpr int kMxRowBytes = kHidden + kPairs; // 6336: MXFP8 output row (E4M3 values + UE8M0 per 32)
constexpr float kRowTarget = 2688.0f;         // 448 * 6

constexpr uint32_t kSentWord = 0x88888888u;   // eight E2M1 -0 nibbles
constexpr uint32_t kSentScale2 = 0xFFFFu;     // two E4M3 NaN bytes with the sign bit set
constexpr uint32_t kSentRow = 0x80000000u;    // -0.0f

// ---------------------------------------------------------------------------------------------
// packed FP32 pairs (sm_100 has .f32x2 arithmetic: one issue slot for two IEEE operations)
// ---------------------------------------------------------------------------------------------
struct F2 { float lo, hi; };

__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) {
  F2 d;
  asm("{ .reg .b64 ra, rb, rd;\n"
      "  mov.b64 ra, {%2, %3}; mov.b64 rb, {%4, %5};\n"
      "  mul.rn.f32x2 rd, ra, rb;\n"
      "  mov.b64 {%0, %1}, rd; }"
      : "=f"(d.lo), "=f"(d.hi) : "f"(a.lo), "f"(a.hi), "f"(b.lo), "f"(b.hi));
  return d;
}
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) {
  F2 d;
  asm("{ .reg .b64 ra, rb, rd;\n"
      "  mov.b64 ra, {%2, %3}; mov.b64 rb, {%4, %5};\n"
      "  add.rn.f32x2 rd, ra, rb;\n"
      "  mov.b64 {%0, %1}, rd; }"
      : "=f"(d.lo), "=f"(d.hi) : "f"(a.lo), "f"(a.hi), "f"(b.lo), "f"(b.hi));
  return d;
}
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
  F2 d;
  asm("{ .reg .b64 ra, rb, rc, rd;\n"
      "  mov.b64 ra, {%2, %3}; mov.b64 rb, {%4, %5}; mov.b64 rc, {%6, %7};\n"
      "  fma.rn.f32x2 rd, ra, rb, rc;\n"
      "  mov.b64 {%0, %1}, rd; }"
      : "=f"(d.lo), "=f"(d.hi) : "f"(a.lo), "f"(a.hi), "f"(b.lo), "f"(b.hi), "f"(c.lo), "f"(c.hi));
  return d;
}
__device__ __forceinline__ F2 f2_splat(float v) { F2 d; d.lo = v; d.hi = v; return d; }

// A 32-bit word holding two BF16 (element 0 in the low half) -> two exact floats.
__device__ __forceinline__ F2 bf16x2_to_f2(uint32_t w) {
  F2 d; d.lo = __uint_as_float(w << 16); d.hi = __uint_as_float(w & 0xffff0000u); return d;
}
// Two floats -> BF16 pair word, round-to-nearest-even (element 0 in the low half).
__device__ __forceinline__ uint32_t f2_to_bf16x2(float lo, float hi) {
  uint32_t w;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
  return w;
}

// ---------------------------------------------------------------------------------------------
// E2M1 / E4M3 conversions
// ---------------------------------------------------------------------------------------------
// Eight floats -> one word of E2M1 nibbles (element 0 in the lowest nibble).  The four result
// bytes are glued as two 16-bit halves inside the asm block; they never exist as separate 8-bit
// C++ values.
__device__ __forceinline__ uint32_t e2m1_pack8(F2 a, F2 b, F2 c, F2 d) {
  uint32_t w;
  asm("{ .reg .b8 q0, q1, q2, q3; .reg .b16 h0, h1;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 q0, %2, %1;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 q1, %4, %3;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 q2, %6, %5;\n"
      "  cvt.rn.satfinite.e2m1x2.f32 q3, %8, %7;\n"
      "  mov.b16 h0, {q0, q1}; mov.b16 h1, {q2, q3};\n"
      "  mov.b32 %0, {h0, h1}; }"
      : "=r"(w)
      : "f"(a.lo), "f"(a.hi), "f"(b.lo), "f"(b.hi), "f"(c.lo), "f"(c.hi), "f"(d.lo), "f"(d.hi));
  return w;
}

// One word of E2M1 nibbles -> eight exact floats (as four pairs).  Each byte is narrowed from a
// shifted 32-bit value: splitting the word with mov.b32 {lo,hi} / mov.b16 {b0,b1} is mis-assembled
// for the upper half by ptxas 12.9 on sm_100a (elements 4 and 5 come out wrong), which the GPU
// codec tests guard against.
__device__ __forceinline__ void e2m1_unpack8(uint32_t w, F2* out) {
  uint32_t h0, h1, h2, h3;
  asm("{ .reg .b8 q0, q1, q2, q3; .reg .b32 t1, t2, t3;\n"
      "  cvt.u8.u32 q0, %4;\n"
      "  shr.u32 t1, %4, 8;  cvt.u8.u32 q1, t1;\n"
      "  shr.u32 t2, %4, 16; cvt.u8.u32 q2, t2;\n"
      "  shr.u32 t3, %4, 24; cvt.u8.u32 q3, t3;\n"
      "  cvt.rn.f16x2.e2m1x2 %0, q0;\n"
      "  cvt.rn.f16x2.e2m1x2 %1, q1;\n"
      "  cvt.rn.f16x2.e2m1x2 %2, q2;\n"
      "  cvt.rn.f16x2.e2m1x2 %3, q3; }"
      : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(w));
  const uint32_t hh[4] = {h0, h1, h2, h3};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&hh[i]));
    out[i].lo = t.x; out[i].hi = t.y;
  }
}

// Two floats -> two E4M3 bytes in the low 16 bits (first value in the low byte).  Block scales feed it
// non-negative numbers; the MXFP8 output feeds it signed ones.
__device__ __forceinline__ uint32_t e4m3_pack2(float first, float second) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(second), "f"(first));
  return r;
}
// Two E4M3 bytes (low 16 bits) -> two exact floats.
__device__ __forceinline__ F2 e4m3_unpack2(uint32_t two) {
  uint32_t h;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(h) : "r"(two));
  const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&h));
  F2 d; d.lo = t.x; d.hi = t.y; return d;
}

// Map every -0 nibble (0x8) to +0 and leave all other nibbles alone.
__device__ __forceinline__ uint32_t canon_neg0(uint32_t w) {
  const uint32_t mag = w & 0x77777777u;                 // magnitude bits of the eight nibbles
  const uint32_t nonzero = mag + 0x77777777u;           // bit 3 of a nibble is set iff its magnitude != 0
  return w & (nonzero | 0x77777777u);                   // keep a sign bit only above a non-zero magnitude
}

// rn(x / 6) for x >= 0, +inf or NaN, without a division: one Newton step on q = x * rn(1/6).
// Differs from IEEE division only where the quotient is subnormal, and every subnormal float
// rounds to the E4M3 byte 0, which is the only consumer.
__device__ __forceinline__ float div6(float x) {
  const float r = 0x1.555556p-3f;
  const float q = __fmul_rn(x, r);
  const float e = __fmaf_rn(-q, 6.0f, x);
  const float q1 = __fmaf_rn(e, r, q);
  return x == __int_as_float(0x7f800000) ? x : q1;
}

// ---------------------------------------------------------------------------------------------
// row scale, block encode, decode-accumulate
// ---------------------------------------------------------------------------------------------
struct RowScale { float inv, rs; };

__device__ __forceinline__ RowScale row_scale_from_amax(float amax) {
  RowScale s;
  s.inv = amax > 0.0f ? __fdiv_rn(kRowTarget, amax) : 0.0f;
  s.rs = __fdiv_rn(amax, kRowTarget);
  return s;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

// max |x| over the eight BF16 of a 16-byte chunk, folded into m (BF16x2 accumulator, lanes independent).
__device__ __forceinline__ __nv_bfloat162 chunk_absmax(uint4 c, __nv_bfloat162 m) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&c);
  m = __hmax2(m, __habs2(p[0])); m = __hmax2(m, __habs2(p[1]));
  m = __hmax2(m, __habs2(p[2])); m = __hmax2(m, __habs2(p[3]));
  return m;
}
// Non-negative BF16 order like unsigned integers: fold the two halves and widen.
__device__ __forceinline__ uint32_t bf16x2_hmax_bits(__nv_bfloat162 m) {
  const uint32_t u = *reinterpret_cast<const uint32_t*>(&m);
  return max(u & 0xffffu, u >> 16);
}

// Scale bytes and value multipliers of the two blocks of one pair.
//   byte = e4m3(rn(rn(blockmax * inv) / 6)),  mult = byte decodes to > 0 ? rn(inv / decode(byte)) : 0
__device__ __forceinline__ uint32_t pair_block_scales(float bm0, float bm1, float inv, float& mult0, float& mult1) {
  const uint32_t sf2 = e4m3_pack2(div6(__fmul_rn(bm0, inv)), div6(__fmul_rn(bm1, inv)));
  const F2 s = e4m3_unpack2(sf2);
  mult0 = s.lo > 0.0f ? __fdiv_rn(inv, s.lo) : 0.0f;
  mult1 = s.hi > 0.0f ? __fdiv_rn(inv, s.hi) : 0.0f;
  return sf2;
}

// The same with a table in shared memory: lut[b] = {decode(b), rn(1 / decode(b))} for the 128 non-negative E4M3
// bytes.  The multiplier rn(inv / decode(b)) is obtained without a division from q0 = rn(inv * rc),
// q1 = fma(fma(-q0, d, inv), rc, q0), which equals the IEEE quotient for every inv in [2^-100, 2^100] and every
// finite positive d of the table (checked exhaustively on the GPU by the test-suite); `exact_ok` says whether
// inv is in that range (the caller computes it once per row), otherwise the IEEE division is used.
struct ScaleLut { const float2* tab; };
__device__ __forceinline__ void fill_scale_lut(float2* tab, int tid, int nthreads) {
  for (int b = tid; b < 128; b += nthreads) {
    const float d = e4m3_unpack2((uint32_t)b).lo;
    tab[b] = make_float2(d, d > 0.0f ? __frcp_rn(d) : 0.0f);
  }
}
__device__ __forceinline__ bool scale_lut_range_ok(float inv) { return inv >= 0x1p-100f && inv <= 0x1p100f; }
__device__ __forceinline__ float lut_multiplier(float inv, float2 e, bool exact_ok) {
  float m;
  if (exact_ok) {
    const float q0 = __fmul_rn(inv, e.y);
    m = __fmaf_rn(__fmaf_rn(-q0, e.x, inv), e.y, q0);
  } else {
    m = __fdiv_rn(inv, e.x);
  }
  return e.x > 0.0f ? m : 0.0f;
}
__device__ __forceinline__ uint32_t pair_block_scales_lut(float bm0, float bm1, float inv, ScaleLut lut, bool exact_ok,
                                                          float& mult0, float& mult1) {
  const uint32_t sf2 = e4m3_pack2(div6(__fmul_rn(bm0, inv)), div6(__fmul_rn(bm1, inv)));
  mult0 = lut_multiplier(inv, lut.tab[sf2 & 0x7fu], exact_ok);
  mult1 = lut_multiplier(inv, lut.tab[(sf2 >> 8) & 0x7fu], exact_ok);
  return sf2;
}

// Eight BF16 (one 16 B chunk) times mult -> E2M1 word.
template <bool CANON>
__device__ __forceinline__ uint32_t quant_chunk_bf16(uint4 c, float mult) {
  const F2 mm = f2_splat(mult);
  const uint32_t w = e2m1_pack8(f2_mul(bf16x2_to_f2(c.x), mm), f2_mul(bf16x2_to_f2(c.y), mm),
                                f2_mul(bf16x2_to_f2(c.z), mm), f2_mul(bf16x2_to_f2(c.w), mm));
  return CANON ? canon_neg0(w) : w;
}

// Eight floats (one 16-byte slot of a pair) times mult -> E2M1 word: the FP32 twin of quant_chunk_bf16.
template <bool CANON>
__device__ __forceinline__ uint32_t quant_slot_f32(const float* v8, float mult) {
  const F2 mm = f2_splat(mult);
  F2 a, b, c, d;
  a.lo = v8[0]; a.hi = v8[1]; b.lo = v8[2]; b.hi = v8[3]; c.lo = v8[4]; c.hi = v8[5]; d.lo = v8[6]; d.hi = v8[7];
  const uint32_t w = e2m1_pack8(f2_mul(a, mm), f2_mul(b, mm), f2_mul(c, mm), f2_mul(d, mm));
  return CANON ? canon_neg0(w) : w;
}
__device__ __forceinline__ float absmax16(const float* f) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; i++) m = fmaxf(m, fabsf(f[i]));
  return m;
}
// Encode a pair held as 32 floats (an FP32 sum re-encoded by the two-shot row owner, or a GEMM accumulator):
// slots 0,1 are the first 16-value block, slots 2,3 the second.  `scales(bm0, bm1, mult0, mult1)` turns the two
// block maxima into the scale bytes (returned) and the value multipliers: pair_block_scales with a row's
// inverse scale, or its table-driven form.
// The form with the two block maxima given is for callers that already have them (for the row maximum).
template <bool CANON, class Scales>
__device__ __forceinline__ uint32_t encode_pair_f32(const float* f, float bm0, float bm1, Scales&& scales, uint4& q) {
  float mult_a, mult_b;
  const uint32_t sf2 = scales(bm0, bm1, mult_a, mult_b);
  q.x = quant_slot_f32<CANON>(f, mult_a);
  q.y = quant_slot_f32<CANON>(f + 8, mult_a);
  q.z = quant_slot_f32<CANON>(f + 16, mult_b);
  q.w = quant_slot_f32<CANON>(f + 24, mult_b);
  return sf2;
}
template <bool CANON, class Scales>
__device__ __forceinline__ uint32_t encode_pair_f32(const float* f, Scales&& scales, uint4& q) {
  return encode_pair_f32<CANON>(f, absmax16(f), absmax16(f + 16), scales, q);
}

__device__ __forceinline__ float absmax32(const float* f, float m) {
#pragma unroll
  for (int i = 0; i < 32; i++) m = fmaxf(m, fabsf(f[i]));
  return m;
}

__device__ __forceinline__ void zero32(float* acc) {
#pragma unroll
  for (int i = 0; i < 32; i++) acc[i] = 0.0f;
}

// 32 floats -> 32 BF16 as four 16 B chunks.
__device__ __forceinline__ void pack32_bf16(const float* f, uint4* c) {
  uint32_t* w = reinterpret_cast<uint32_t*>(c);
#pragma unroll
  for (int i = 0; i < 16; i++) w[i] = f2_to_bf16x2(f[2 * i], f[2 * i + 1]);
}

// ---------------------------------------------------------------------------------------------
// receive-side validity (Lamport-in-data): a field is "not yet written" while it still holds a sentinel
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool values_pending(uint4 q) {
  return (q.x == kSentWord) | (q.y == kSentWord) | (q.z == kSentWord) | (q.w == kSentWord);
}
__device__ __forceinline__ bool scales_pending(uint32_t sf2) { return (sf2 & 0x8080u) != 0; }
__device__ __forceinline__ bool rowscale_pending(uint32_t bits) { return bits == kSentRow; }

// ---------------------------------------------------------------------------------------------
// Gemma RMSNorm epilogue:  z = sum + residual, res_out = bf16(z),
//   y = (bf16(z) * rinv) * (wbias + w),  rinv = 1 / sqrt(sumsq(z) / 6144 + eps)   (all IEEE rn)
// Reference project: kernels/fused_norm/lnorm_epi.cuh:23-70; its approximate rsqrt is replaced by
// exact operations so that the host model can reproduce the result.
// ---------------------------------------------------------------------------------------------
// z (in place in acc) and the pair's sum of squares.  Per 8-value chunk the even and the odd elements
// are accumulated separately in element order and added; the four chunk sums are combined as
// (t0 + t1) + (t2 + t3), which is the same number for every order in which a lane may hold its chunks.
__device__ __forceinline__ float add_residual_sumsq(float* acc, const uint4* res) {
  const uint32_t* rw = reinterpret_cast<const uint32_t*>(res);
  float t[4];
#pragma unroll
  for (int c = 0; c < 4; c++) {
    F2 ss = f2_splat(0.0f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      F2 a; a.lo = acc[8 * c + 2 * i]; a.hi = acc[8 * c + 2 * i + 1];
      a = f2_add(a, bf16x2_to_f2(rw[4 * c + i]));
      ss = f2_fma(a, a, ss);
      acc[8 * c + 2 * i] = a.lo; acc[8 * c + 2 * i + 1] = a.hi;
    }
    t[c] = __fadd_rn(ss.lo, ss.hi);
  }
  return __fadd_rn(__fadd_rn(t[0], t[1]), __fadd_rn(t[2], t[3]));
}
__device__ __forceinline__ float warp_sum_butterfly(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
__device__ __forceinline__ float norm_rinv(float sumsq, float eps) {
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, (float)kHidden), eps)));
}
// y for one pair from BF16 z (4 chunks) and BF16 weights (4 chunks).
__device__ __forceinline__ void norm_pair(const uint4* zb, const uint4* wt, float rinv, float wbias, float* y) {
  const uint32_t* zw = reinterpret_cast<const uint32_t*>(zb);
  const uint32_t* ww = reinterpret_cast<const uint32_t*>(wt);
  const F2 r2 = f2_splat(rinv), b2 = f2_splat(wbias);
#pragma unroll
  for (int i = 0; i < 16; i++) {
    const F2 t = f2_mul(f2_mul(bf16x2_to_f2(zw[i]), r2), f2_add(b2, bf16x2_to_f2(ww[i])));
    y[2 * i] = t.lo; y[2 * i + 1] = t.hi;
  }
}
// NVFP4 output of one pair of BF16-rounded y: s = e4m3(gsc * (blockmax / 6)), q = e2m1(y * rn(gsc / e4m3(s))).
// No -0 canonicalisation (this is a tensor for a GEMM, not a receive window).  Returns the two scale bytes.
__device__ __forceinline__ uint32_t quant_pair_nvfp4_out(const uint4* yb, float gsc, uint4& q) {
  const __nv_bfloat162 z2 = __floats2bfloat162_rn(0.0f, 0.0f);
  const float bm0 = __uint_as_float(bf16x2_hmax_bits(chunk_absmax(yb[1], chunk_absmax(yb[0], z2))) << 16);
  const float bm1 = __uint_as_float(bf16x2_hmax_bits(chunk_absmax(yb[3], chunk_absmax(yb[2], z2))) << 16);
  const uint32_t sf2 = e4m3_pack2(__fmul_rn(gsc, div6(bm0)), __fmul_rn(gsc, div6(bm1)));
  const F2 s = e4m3_unpack2(sf2);
  const float o0 = s.lo != 0.0f ? __fdiv_rn(gsc, s.lo) : 0.0f;
  const float o1 = s.hi != 0.0f ? __fdiv_rn(gsc, s.hi) : 0.0f;
  q.x = quant_chunk_bf16<false>(yb[0], o0); q.y = quant_chunk_bf16<false>(yb[1], o0);
  q.z = quant_chunk_bf16<false>(yb[2], o1); q.w = quant_chunk_bf16<false>(yb[3], o1);
  return sf2;
}
// MXFP8 output of one pair (= one 32-block) of BF16-rounded y: UE8M0 scale e = clamp(ceil(log2(amax/448)) + 127),
// values e4m3(y * 2^(127-e)).  v[0..1] receive the 32 value bytes; returns the scale byte.
__device__ __forceinline__ uint32_t quant_pair_mxfp8_out(const uint4* yb, uint4* v) {
  __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
  for (int k = 0; k < 4; k++) m2 = chunk_absmax(yb[k], m2);
  float am = __uint_as_float(bf16x2_hmax_bits(m2) << 16);
  am = fmaxf(am, 1.17549435e-38f);
  const uint32_t qb = __float_as_uint(__fdiv_rn(am, 448.0f));
  const int ef = (int)((qb >> 23) & 0xffu);
  int ce = ef - 127 + ((qb & 0x7fffffu) ? 1 : 0);
  if (ef == 0) ce = -126;
  int e = ce + 127;
  e = e < 0 ? 0 : (e > 254 ? 254 : e);
  const float mult = e == 254 ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(254 - e) << 23);
  const uint32_t* yw = reinterpret_cast<const uint32_t*>(yb);
  uint32_t w[8];
  const F2 mm = f2_splat(mult);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const F2 a = f2_mul(bf16x2_to_f2(yw[2 * i]), mm), b = f2_mul(bf16x2_to_f2(yw[2 * i + 1]), mm);
    w[i] = e4m3_pack2(a.lo, a.hi) | (e4m3_pack2(b.lo, b.hi) << 16);
  }
  v[0] = make_uint4(w[0], w[1], w[2], w[3]);
  v[1] = make_uint4(w[4], w[5], w[6], w[7]);
  return (uint32_t)e;
}

}  // namespace fp4ar
