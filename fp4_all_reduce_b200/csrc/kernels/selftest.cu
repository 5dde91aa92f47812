// Exhaustive device self-tests of the conversion primitives the codec is built on, each against a plain software
// model written out below (thresholds and bit arithmetic, no special instructions):
//
//   block scale   every non-negative FP32 x (and NaN): cvt.rn.satfinite.e4m3x2.f32(div6(x)) == soft_e4m3(x / 6)
//                 with an IEEE division; covers the division-free div6 and the hardware E4M3 rounding
//   value         every FP32 bit pattern: the nibble of cvt.rn.satfinite.e2m1x2.f32 == soft_e2m1(x), in each of the
//                 eight positions of e2m1_pack8
//   decode        every 16-bit pattern in either half of a word through e2m1_unpack8, every pair of scale bytes
//                 through e4m3_unpack2, against tables; canon_neg0 on every 16-bit pattern in either half
//   pairs         2^28 pseudo-random BF16 pairs and 2^26 FP32 pairs (normal, tiny, narrow-band and mostly-zero classes):
//                 the table-driven block encoder equals the one with IEEE divisions and never produces a sentinel
//                 (value word 0x88888888, scale byte with the top bit set, row scale -0); 2^28 decode-accumulate cases
//                 over every pair of scale bytes against scalar table arithmetic
//
// Each kernel adds its mismatch count to a counter; the host test expects 0.  Nothing here can fault: the kernels
// only convert numbers held in registers.
//
// Reference project counterparts: tests T1, T3-T5 of bench/codec/codec_bench.cu:29-134 and tests/codec_test.cu:31-72.
#include <cuda_runtime.h>
#include <cmath>
#include <cstring>
#include "../include/fp4ar.h"
#include "../include/fp4ar_codec.cuh"
#include "host_util.h"

namespace fp4ar {

__host__ __device__ inline uint32_t soft_e4m3(float x) {   // x >= 0 or NaN
  if (x != x) return 0x7fu;
  if (x >= 448.0f) return 0x7eu;
  if (x < 0x1p-6f) return (uint32_t)rintf(x * 512.0f);     // subnormal grid, step 2^-9; 8 is the first normal
  int e;
  const float m = frexpf(x, &e);                           // x = m * 2^e, m in [0.5, 1)
  int q = (int)rintf((2.0f * m - 1.0f) * 8.0f);
  int E = e - 1;
  if (q == 8) { q = 0; E += 1; }
  const int byte = ((E + 7) << 3) | q;
  return (uint32_t)(byte > 0x7e ? 0x7e : byte);
}

__host__ __device__ inline uint32_t soft_e2m1(float x) {
  if (x != x) return 7u;
  const uint32_t sign = signbit(x) ? 8u : 0u;
  const float a = fabsf(x);
  uint32_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return sign | c;
}

__host__ __device__ inline float soft_e2m1_value(uint32_t n) {
  const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const float v = mag[n & 7u];
  return (n & 8u) ? -v : v;
}
__host__ __device__ inline float soft_e4m3_value(uint32_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  float v = e ? ldexpf(1.0f + m / 8.0f, e - 7) : ldexpf(m / 8.0f, -6);
  return (b & 0x80u) ? -v : v;
}

// u runs over [first, first + count) of non-negative FP32 bit patterns (0 .. 0x7fffffff: finite, +inf, NaNs)
__global__ void selftest_block_scale_kernel(uint32_t first, uint32_t count, unsigned long long* mismatches) {
  unsigned long long bad = 0;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
    const float x = __uint_as_float(first + i);
    const uint32_t hw = e4m3_pack2(div6(x), 0.0f) & 0xffu;
    const uint32_t sw = soft_e4m3(__fdiv_rn(x, 6.0f));
    bad += hw != sw;
  }
  if (bad) atomicAdd(mismatches, bad);
}

// every FP32 bit pattern of [first, first + count), in nibble position (pattern & 7) of the packed word
__global__ void selftest_e2m1_encode_kernel(uint32_t first, uint32_t count, unsigned long long* mismatches) {
  unsigned long long bad = 0;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
    const uint32_t u = first + i;
    const float x = __uint_as_float(u);
    const int pos = (int)(u & 7u);
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = (k == pos) ? x : 1.0f;      // 1.0 encodes as nibble 2 everywhere else
    F2 a, b, c, d;
    a.lo = v[0]; a.hi = v[1]; b.lo = v[2]; b.hi = v[3]; c.lo = v[4]; c.hi = v[5]; d.lo = v[6]; d.hi = v[7];
    const uint32_t w = e2m1_pack8(a, b, c, d);
    uint32_t want = 0x22222222u;
    want = (want & ~(0xfu << (4 * pos))) | (soft_e2m1(x) << (4 * pos));
    bad += w != want;
  }
  if (bad) atomicAdd(mismatches, bad);
}

// 2 x 65536 value words, 65536 scale pairs, 2 x 65536 canonicalisations
__global__ void selftest_decode_kernel(unsigned long long* mismatches) {
  unsigned long long bad = 0;
  for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < 65536u; p += gridDim.x * blockDim.x) {
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const uint32_t w = half ? ((p << 16) | 0x2222u) : (p | 0x22220000u);
      F2 out[4];
      e2m1_unpack8(w, out);
      const float got[8] = {out[0].lo, out[0].hi, out[1].lo, out[1].hi, out[2].lo, out[2].hi, out[3].lo, out[3].hi};
#pragma unroll
      for (int k = 0; k < 8; k++) bad += __float_as_uint(got[k]) != __float_as_uint(soft_e2m1_value((w >> (4 * k)) & 15u));
      // canonicalisation: every -0 nibble becomes +0, nothing else changes
      uint32_t want = w;
#pragma unroll
      for (int k = 0; k < 8; k++)
        if (((w >> (4 * k)) & 15u) == 8u) want &= ~(0xfu << (4 * k));
      bad += canon_neg0(w) != want;
    }
    const F2 s = e4m3_unpack2(p);
    const uint32_t b0 = p & 0xffu, b1 = p >> 8;
    const float w0 = soft_e4m3_value(b0), w1 = soft_e4m3_value(b1);
    if ((b0 & 0x7fu) == 0x7fu) bad += !(s.lo != s.lo); else bad += __float_as_uint(s.lo) != __float_as_uint(w0);
    if ((b1 & 0x7fu) == 0x7fu) bad += !(s.hi != s.hi); else bad += __float_as_uint(s.hi) != __float_as_uint(w1);
  }
  if (bad) atomicAdd(mismatches, bad);
}


// ---- pair-level tests on pseudo-random inputs (counter-based hash, so a run is reproducible from its seed) ----
__host__ __device__ inline uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
// A BF16 bit pattern for test class `cls`: 0 any finite value, 1 tiny / subnormal magnitudes, 2 a narrow band around 1,
// 3 mostly zeros (+0 and -0) with a few values.
__device__ __forceinline__ uint32_t test_bf16(uint32_t h, int cls) {
  uint32_t b = h & 0xffffu;
  if ((b & 0x7f80u) == 0x7f80u) b &= 0xbfffu;                       // no inf / NaN
  if (cls == 1) b = (b & 0x807fu) | (((h >> 16) & 7u) << 7);        // exponents 0..7
  else if (cls == 2) b = (b & 0x807fu) | ((126u + ((h >> 16) & 3u)) << 7);
  else if (cls == 3) { if ((h >> 20) & 7u) b &= 0x8000u; }
  return b;
}

// One pair per thread and iteration: 32 BF16 values and a row-scale inverse no smaller than the pair needs.
//   the encoder with the table-driven multipliers  ==  the encoder with IEEE divisions, word for word;
//   no value word equals the value sentinel and no scale byte has its top bit set (counter[1]).
__global__ void selftest_pair_bf16_kernel(uint32_t seed, uint32_t count, unsigned long long* counters) {
  __shared__ float2 tab[128];
  fill_scale_lut(tab, threadIdx.x, blockDim.x);
  __syncthreads();
  const ScaleLut lut{tab};
  unsigned long long bad = 0, sent = 0;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
    const int cls = (int)(i & 3u);
    uint4 c[4];
    uint32_t* w = reinterpret_cast<uint32_t*>(c);
    float am = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; k++) {
      const uint32_t h = mix32(seed ^ mix32(i * 16u + (uint32_t)k));
      const uint32_t lo = test_bf16(h, cls), hi = test_bf16(mix32(h), cls);
      w[k] = lo | (hi << 16);
      am = fmaxf(am, fmaxf(fabsf(__uint_as_float(lo << 16)), fabsf(__uint_as_float(hi << 16))));
    }
    // the row maximum is at least the pair's; sometimes much larger (the pair then encodes to small codes)
    const float row_am = am * __uint_as_float(0x3f800000u + ((mix32(i ^ seed) & 0x1fu) << 23));
    const RowScale sc = row_scale_from_amax(row_am);
    const __nv_bfloat162 z2 = __floats2bfloat162_rn(0.0f, 0.0f);
    const float bm0 = __uint_as_float(bf16x2_hmax_bits(chunk_absmax(c[1], chunk_absmax(c[0], z2))) << 16);
    const float bm1 = __uint_as_float(bf16x2_hmax_bits(chunk_absmax(c[3], chunk_absmax(c[2], z2))) << 16);
    float a0, a1, b0, b1;
    const uint32_t sfa = pair_block_scales(bm0, bm1, sc.inv, a0, a1);
    const uint32_t sfb = pair_block_scales_lut(bm0, bm1, sc.inv, lut, scale_lut_range_ok(sc.inv), b0, b1);
    bad += sfa != sfb;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint32_t qa = quant_chunk_bf16<true>(c[k], k < 2 ? a0 : a1);
      const uint32_t qb = quant_chunk_bf16<true>(c[k], k < 2 ? b0 : b1);
      bad += qa != qb;
      sent += qb == kSentWord;
    }
    sent += (sfb & 0x8080u) != 0u;
    sent += __float_as_uint(sc.rs) == kSentRow;
  }
  if (bad) atomicAdd(counters, bad);
  if (sent) atomicAdd(counters + 1, sent);
}

// The same for a pair held as 32 floats (the two-shot owner's re-encode): table-driven == IEEE, no sentinel.
__global__ void selftest_pair_f32_kernel(uint32_t seed, uint32_t count, unsigned long long* counters) {
  __shared__ float2 tab[128];
  fill_scale_lut(tab, threadIdx.x, blockDim.x);
  __syncthreads();
  const ScaleLut lut{tab};
  unsigned long long bad = 0, sent = 0;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
    float f[32];
    float am = 0.0f;
#pragma unroll
    for (int k = 0; k < 32; k++) {
      uint32_t h = mix32(seed ^ mix32(i * 32u + (uint32_t)k));
      if ((h & 0x7f800000u) == 0x7f800000u) h &= 0xbfffffffu;       // finite
      if ((i & 3u) == 1u) h = (h & 0x807fffffu) | (((h >> 3) & 15u) << 23);   // tiny magnitudes
      if ((i & 3u) == 3u && (h & 0x700u)) h &= 0x80000000u;         // mostly +-0
      f[k] = __uint_as_float(h);
      am = fmaxf(am, fabsf(f[k]));
    }
    const float row_am = am * __uint_as_float(0x3f800000u + ((mix32(i ^ seed) & 0xfu) << 23));
    const RowScale sc = row_scale_from_amax(row_am);
    const bool ok = scale_lut_range_ok(sc.inv);
    uint4 qa, qb;
    const uint32_t sfa = encode_pair_f32<true>(f, [&](float x0, float x1, float& m0, float& m1) { return pair_block_scales(x0, x1, sc.inv, m0, m1); }, qa);
    const uint32_t sfb = encode_pair_f32<true>(f, [&](float x0, float x1, float& m0, float& m1) { return pair_block_scales_lut(x0, x1, sc.inv, lut, ok, m0, m1); }, qb);
    bad += (sfa != sfb) + (qa.x != qb.x) + (qa.y != qb.y) + (qa.z != qb.z) + (qa.w != qb.w);
    sent += (qb.x == kSentWord) + (qb.y == kSentWord) + (qb.z == kSentWord) + (qb.w == kSentWord) + ((sfb & 0x8080u) != 0u);
  }
  if (bad) atomicAdd(counters, bad);
  if (sent) atomicAdd(counters + 1, sent);
}

// Decode-accumulate: for every pair of scale bytes (all 2^14 non-negative combinations), pseudo-random value words,
// row scales and starting sums, the packed f32x2 path equals scalar  fmaf(e2m1, rn(e4m3 * rs), acc)  from the tables.
__global__ void selftest_decode_acc_kernel(uint32_t seed, uint32_t reps, unsigned long long* counters) {
  unsigned long long bad = 0;
  const uint32_t total = reps << 14;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const uint32_t sf2 = (i & 0x7fu) | (((i >> 7) & 0x7fu) << 8);
    if ((sf2 & 0x7fu) == 0x7fu || (sf2 >> 8) == 0x7fu) continue;    // the NaN byte decodes to NaN, whose payload is not pinned down: the table test covers it
    const uint32_t h = mix32(seed ^ mix32(i));
    uint4 q;
    q.x = canon_neg0(h); q.y = canon_neg0(mix32(h + 1u)); q.z = canon_neg0(mix32(h + 2u)); q.w = canon_neg0(mix32(h + 3u));
    const float rs = __uint_as_float(0x30000000u + (mix32(h + 4u) & 0x1fffffffu));   // 2^-31 .. 2^33
    float acc[32], ref[32];
#pragma unroll
    for (int k = 0; k < 32; k++) { acc[k] = __uint_as_float(0x3c000000u + (mix32(h + 8u + k) & 0x87ffffffu)); ref[k] = acc[k]; }
    {
      const F2 e = e4m3_unpack2(sf2);
      const F2 sa = f2_splat(__fmul_rn(e.lo, rs)), sb = f2_splat(__fmul_rn(e.hi, rs));
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; k++) {
        F2 v[4];
        e2m1_unpack8(w[k], v);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          F2 a; a.lo = acc[8 * k + 2 * j]; a.hi = acc[8 * k + 2 * j + 1];
          a = f2_fma(v[j], k < 2 ? sa : sb, a);
          acc[8 * k + 2 * j] = a.lo; acc[8 * k + 2 * j + 1] = a.hi;
        }
      }
    }
    const float s0 = __fmul_rn(soft_e4m3_value(sf2 & 0xffu), rs), s1 = __fmul_rn(soft_e4m3_value(sf2 >> 8), rs);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 32; k++) {
      const float v = soft_e2m1_value((w[k >> 3] >> (4 * (k & 7))) & 15u);
      ref[k] = __fmaf_rn(v, k < 16 ? s0 : s1, ref[k]);
      bad += __float_as_uint(ref[k]) != __float_as_uint(acc[k]);
    }
  }
  if (bad) atomicAdd(counters, bad);
}

}  // namespace fp4ar

using namespace fp4ar;

// which: 0 block scale (patterns 0 .. 0x7fffffff), 1 value encode (all 2^32 patterns), 2 decode / canonicalise tables.
// For 0 and 1 the range [first, first + count) is tested (count 0 = up to the end of the domain).
// which 3, 4, 5: pair-level tests on `count` pseudo-random cases with seed `first` (3: BF16 pairs, 4: FP32 pairs: the
// table-driven encoder equals the IEEE-division encoder and never emits a sentinel, counter[1]; 5: decode-accumulate
// against scalar table arithmetic for every pair of scale bytes, `count` rounds of 2^14 cases).
extern "C" int fp4ar_selftest_conversions(int which, unsigned int first, unsigned int count,
                                          unsigned long long* device_mismatch_counter, fp4ar_stream stream) {
  if (!device_mismatch_counter || which < 0 || which > 5) return FP4AR_ERR_ARGUMENT;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = 8 * device_sm_count();
  if (which == 0) {
    if (first > 0x7fffffffu) return FP4AR_ERR_ARGUMENT;
    const unsigned int room = 0x80000000u - first;
    if (count == 0 || count > room) count = room;
    selftest_block_scale_kernel<<<grid, 256, 0, st>>>(first, count, device_mismatch_counter);
  } else if (which == 1) {
    const unsigned long long room = 0x100000000ull - first;
    if (count == 0 || count > room) count = (unsigned int)(room > 0xffffffffull ? 0xffffffffull : room);
    selftest_e2m1_encode_kernel<<<grid, 256, 0, st>>>(first, count, device_mismatch_counter);
  } else if (which == 2) {
    selftest_decode_kernel<<<256, 256, 0, st>>>(device_mismatch_counter);
  } else if (which == 3) {
    selftest_pair_bf16_kernel<<<grid, 256, 0, st>>>(first, count, device_mismatch_counter);
  } else if (which == 4) {
    selftest_pair_f32_kernel<<<grid, 256, 0, st>>>(first, count, device_mismatch_counter);
  } else {
    if (count > (1u << 17)) return FP4AR_ERR_ARGUMENT;
    selftest_decode_acc_kernel<<<grid, 256, 0, st>>>(first, count, device_mismatch_counter);
  }
  return cuda_check_launch();
}

// The software models themselves, callable on the host, so that they can be checked against the host model of the
// codec without a GPU.  what: 0 soft_e4m3 (x >= 0 or NaN), 1 soft_e2m1, 2 soft_e2m1_value, 3 soft_e4m3_value.
extern "C" int fp4ar_selftest_soft_model(int what, const float* in, const unsigned int* in_bits, int n, unsigned int* out_bits) {
  if (n < 0 || !out_bits) return FP4AR_ERR_ARGUMENT;
  for (int i = 0; i < n; i++) {
    switch (what) {
      case 0: out_bits[i] = soft_e4m3(in[i]); break;
      case 1: out_bits[i] = soft_e2m1(in[i]); break;
      case 2: { const float v = soft_e2m1_value(in_bits[i]); memcpy(&out_bits[i], &v, 4); break; }
      case 3: { const float v = soft_e4m3_value(in_bits[i]); memcpy(&out_bits[i], &v, 4); break; }
      default: return FP4AR_ERR_ARGUMENT;
    }
  }
  return FP4AR_OK;
}
