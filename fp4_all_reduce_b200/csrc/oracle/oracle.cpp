// Host-only bit-exact model of the NVFP4 row transport ("codec spec v2") and of every fused
// operator built on it.  Nothing here shares code with the device kernels: the kernels are
// gated bit for bit against this file, and this file is gated against an independent numpy
// model in the test-suite.
//
// Parity with the reference project: the arithmetic follows include/fp4_codec.cuh:82-133
// (row scale, block scale, value quantisation, decode-accumulate), harness/ref.cuh:54-88
// (one-shot / two-shot references), harness/ref.cuh:144-190 (static-scale NVFP4 input) and
// kernels/fused_norm/lnorm_epi.cuh:61-118 (Gemma RMSNorm epilogue, NVFP4 / MXFP8 quantisers).
// Deviation, on purpose: the norm epilogue uses IEEE round-to-nearest division and square root
// where the reference uses the GPU's approximate rsqrt / rcp, so that a host can reproduce it.
//
// Build: g++ -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC oracle.cpp
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>

namespace {

constexpr int H = 6144;          // hidden size of one row
constexpr int VB = H / 2;        // E2M1 value bytes per row
constexpr int SB = H / 16;       // E4M3 block-scale bytes per row
constexpr int NBLK = H / 16;     // 16-value blocks per row
constexpr int PAIRS = H / 32;    // 32-value pairs per row
constexpr float ROW_TARGET = 2688.0f;  // 448 (largest E4M3) * 6 (largest E2M1)

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

inline float bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

// Round-to-nearest-even; every NaN becomes the canonical 0x7FFF the GPU conversion produces.
inline uint16_t f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// ---- E4M3 (finite-only format: 0x7F is NaN, largest finite 0x7E = 448) ----
float g_e4m3_val[256];
float g_e2m1_val[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

struct TableInit {
  TableInit() {
    for (int b = 0; b < 256; b++) {
      const int e = (b >> 3) & 15, m = b & 7;
      float v = e ? std::ldexp(1.0f + m / 8.0f, e - 7) : std::ldexp(m / 8.0f, -6);
      if ((b & 0x7f) == 0x7f) v = NAN;
      g_e4m3_val[b] = (b & 0x80) ? -v : v;
    }
  }
} g_table_init;

// float -> E4M3 byte, round-to-nearest-even, saturating to +-448; NaN -> 0x7F.
inline uint8_t e4m3_encode(float x) {
  if (std::isnan(x)) return 0x7f;
  const uint8_t sign = std::signbit(x) ? 0x80 : 0;
  const float a = std::fabs(x);
  if (a >= 448.0f) return sign | 0x7e;
  if (a < 0.015625f) {  // below 2^-6: subnormal grid of step 2^-9 (a value of 8 is the first normal)
    const int q = (int)std::nearbyint(std::ldexp(a, 9));
    return sign | (uint8_t)q;
  }
  int e;
  const float m = std::frexp(a, &e);          // a = m * 2^e, m in [0.5, 1)
  int q = (int)std::nearbyint((2.0f * m - 1.0f) * 8.0f);
  int E = e - 1;
  if (q == 8) { q = 0; E += 1; }
  int byte = ((E + 7) << 3) | q;
  if (byte > 0x7e) byte = 0x7e;
  return sign | (uint8_t)byte;
}

// float -> E2M1 nibble, round-to-nearest-even on the grid {0,.5,1,1.5,2,3,4,6}, saturating;
// NaN -> 0x7 (+6), which is what cvt.rn.satfinite.e2m1x2.f32 does.
inline uint8_t e2m1_encode(float x) {
  if (std::isnan(x)) return 7;
  const uint8_t sign = std::signbit(x) ? 8 : 0;
  const float a = std::fabs(x);
  uint8_t c;
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

inline float absmax(const float* f, int n) {
  float m = 0.f;
  for (int i = 0; i < n; i++) { const float a = std::fabs(f[i]); if (a > m) m = a; }  // NaN never wins
  return m;
}

// One row (H floats) -> values v[VB], scales s[SB]. `inv` is the multiplier applied before the
// block scale is taken (2688/amax for the dynamic row scale, 1/gs for a static one).
void encode_row_with_inv(const float* f, float inv, uint8_t* v, uint8_t* s, bool canon) {
  for (int b = 0; b < NBLK; b++) {
    const float bm = absmax(f + 16 * b, 16);
    const float sv = (bm * inv) / 6.0f;
    const uint8_t sb = e4m3_encode(sv);
    s[b] = sb;
    const float sff = g_e4m3_val[sb];
    const float m = sff > 0.f ? inv / sff : 0.f;
    for (int i = 0; i < 16; i += 2) {
      uint8_t n0 = e2m1_encode(f[16 * b + i] * m), n1 = e2m1_encode(f[16 * b + i + 1] * m);
      if (canon) { if (n0 == 8) n0 = 0; if (n1 == 8) n1 = 0; }
      v[(16 * b + i) >> 1] = (uint8_t)(n0 | (n1 << 4));
    }
  }
}

float encode_row_dynamic(const float* f, uint8_t* v, uint8_t* s, bool canon) {
  const float am = absmax(f, H);
  const float inv = am > 0.f ? ROW_TARGET / am : 0.f;
  encode_row_with_inv(f, inv, v, s, canon);
  return am / ROW_TARGET;
}

void decode_acc_row(float* acc, const uint8_t* v, const uint8_t* s, float rs) {
  for (int b = 0; b < NBLK; b++) {
    const float S = g_e4m3_val[s[b]] * rs;
    for (int i = 0; i < 16; i++) {
      const int n = (v[(16 * b + i) >> 1] >> (4 * (i & 1))) & 15;
      acc[16 * b + i] = std::fmaf(g_e2m1_val[n], S, acc[16 * b + i]);
    }
  }
}

// Sum of squares of one row in the fixed order every kernel reproduces:
//   chunk c of a pair (8 values): e = fma over its even elements in order, o = fma over its odd elements, t_c = e + o
//   pair p (32 values = chunks 0..3): s_p = (t_0 + t_1) + (t_2 + t_3)
//     (a tree that does not change when chunks 0<->1 / 2<->3 or the halves are swapped, which lets a
//      kernel keep the chunks of a pair in any of its four lane-dependent orders)
//   group j (pairs 32j..32j+31): butterfly over the 32 pair sums with partner distance 16,8,4,2,1
//   row: ((((G0 + G1) + G2) + G3) + G4) + G5
float row_sumsq(const float* z) {
  float G[6];
  for (int j = 0; j < 6; j++) {
    float t[32];
    for (int l = 0; l < 32; l++) {
      const float* p = z + 32 * (l + 32 * j);
      float tc[4];
      for (int c = 0; c < 4; c++) {
        float e = 0.f, o = 0.f;
        for (int i = 0; i < 4; i++) {
          e = std::fmaf(p[8 * c + 2 * i], p[8 * c + 2 * i], e);
          o = std::fmaf(p[8 * c + 2 * i + 1], p[8 * c + 2 * i + 1], o);
        }
        tc[c] = e + o;
      }
      t[l] = (tc[0] + tc[1]) + (tc[2] + tc[3]);
    }
    for (int d = 16; d; d >>= 1) {
      float u[32];
      for (int l = 0; l < 32; l++) u[l] = t[l] + t[l ^ d];
      std::memcpy(t, u, sizeof(t));
    }
    G[j] = t[0];
  }
  float ss = G[0];
  for (int j = 1; j < 6; j++) ss = ss + G[j];
  return ss;
}

// NVFP4 output of the norm epilogue for one row of BF16-rounded y (values first, then scales).
void quant_row_nvfp4_out(const float* yb, float gsc, uint8_t* v, uint8_t* s) {
  for (int b = 0; b < NBLK; b++) {
    const float vm = absmax(yb + 16 * b, 16);
    const float sfv = gsc * (vm / 6.0f);
    const uint8_t sb = e4m3_encode(sfv);
    s[b] = sb;
    const float sff = g_e4m3_val[sb];
    const float os = sff != 0.f ? gsc / sff : 0.f;   // NaN scale (never reached with finite input) gives NaN
    for (int i = 0; i < 16; i += 2) {
      const uint8_t n0 = e2m1_encode(yb[16 * b + i] * os), n1 = e2m1_encode(yb[16 * b + i + 1] * os);
      v[(16 * b + i) >> 1] = (uint8_t)(n0 | (n1 << 4));
    }
  }
}

// MXFP8 output: E4M3 values with one UE8M0 scale per 32 values.
void quant_row_mxfp8_out(const float* yb, uint8_t* v, uint8_t* s) {
  for (int p = 0; p < PAIRS; p++) {
    float am = absmax(yb + 32 * p, 32);
    if (am < 1.17549435e-38f) am = 1.17549435e-38f;
    const uint32_t qb = f2u(am / 448.0f);
    const int ef = (int)((qb >> 23) & 0xff);
    int ce = ef - 127 + ((qb & 0x7fffffu) ? 1 : 0);
    if (ef == 0) ce = -126;
    int e = ce + 127;
    e = e < 0 ? 0 : (e > 254 ? 254 : e);
    const float m = e == 254 ? u2f(0x00400000u) : u2f((uint32_t)(254 - e) << 23);
    for (int i = 0; i < 32; i++) v[32 * p + i] = e4m3_encode(yb[32 * p + i] * m);
    s[p] = (uint8_t)e;
  }
}

}  // namespace

extern "C" {

int fp4ar_oracle_hidden() { return H; }

// ---- scalar primitives (exposed for exhaustive tests) ----
uint8_t fp4ar_oracle_e4m3_encode(float x) { return e4m3_encode(x); }
float fp4ar_oracle_e4m3_decode(uint8_t b) { return g_e4m3_val[b]; }
uint8_t fp4ar_oracle_e2m1_encode(float x) { return e2m1_encode(x); }
float fp4ar_oracle_e2m1_decode(uint8_t n) { return g_e2m1_val[n & 15]; }
uint16_t fp4ar_oracle_bf16_rn(float x) { return f32_to_bf16(x); }

void fp4ar_oracle_e4m3_encode_n(const float* x, uint8_t* out, long n) {
#pragma omp parallel for
  for (long i = 0; i < n; i++) out[i] = e4m3_encode(x[i]);
}
void fp4ar_oracle_e2m1_encode_n(const float* x, uint8_t* out, long n) {
#pragma omp parallel for
  for (long i = 0; i < n; i++) out[i] = e2m1_encode(x[i]);
}

// ---- row codec ----
// x: [rows][H] BF16 bits.  v: [rows][3072], s: [rows][384], rs: [rows].  Strides in bytes.
void fp4ar_oracle_encode(const uint16_t* x, int rows, uint8_t* v, long v_stride, uint8_t* s, long s_stride,
                         float* rs, int canon) {
#pragma omp parallel for
  for (int r = 0; r < rows; r++) {
    std::vector<float> f(H);
    for (int i = 0; i < H; i++) f[i] = bf16_to_f32(x[(size_t)r * H + i]);
    rs[r] = encode_row_dynamic(f.data(), v + (size_t)r * v_stride, s + (size_t)r * s_stride, canon != 0);
  }
}

// FP32 input rows (the two-shot owner's re-encode of an FP32 sum).
void fp4ar_oracle_encode_f32(const float* x, int rows, uint8_t* v, long v_stride, uint8_t* s, long s_stride,
                             float* rs, int canon) {
#pragma omp parallel for
  for (int r = 0; r < rows; r++)
    rs[r] = encode_row_dynamic(x + (size_t)r * H, v + (size_t)r * v_stride, s + (size_t)r * s_stride, canon != 0);
}

// Static per-tensor scale gs: inv = rn(1/gs), no row scale on the wire, -0 canonicalised.
void fp4ar_oracle_encode_static(const uint16_t* x, int rows, float gs, uint8_t* v, long v_stride, uint8_t* s,
                                long s_stride) {
  const float inv = 1.0f / gs;
#pragma omp parallel for
  for (int r = 0; r < rows; r++) {
    std::vector<float> f(H);
    for (int i = 0; i < H; i++) f[i] = bf16_to_f32(x[(size_t)r * H + i]);
    encode_row_with_inv(f.data(), inv, v + (size_t)r * v_stride, s + (size_t)r * s_stride, true);
  }
}

// FP32 rows with a static scale (what the GEMM epilogue does to its accumulators); `cols` per row, multiple of 16.
void fp4ar_oracle_encode_static_f32(const float* x, int rows, int cols, float gs, uint8_t* v, long v_stride, uint8_t* s,
                                    long s_stride) {
  const float inv = 1.0f / gs;
#pragma omp parallel for
  for (int r = 0; r < rows; r++) {
    const float* f = x + (size_t)r * cols;
    uint8_t* vr = v + (size_t)r * v_stride;
    uint8_t* sr = s + (size_t)r * s_stride;
    for (int b = 0; b < cols / 16; b++) {
      const float bm = absmax(f + 16 * b, 16);
      const uint8_t sb = e4m3_encode((bm * inv) / 6.0f);
      sr[b] = sb;
      const float sff = g_e4m3_val[sb];
      const float m = sff > 0.f ? inv / sff : 0.f;
      for (int i = 0; i < 16; i += 2) {
        uint8_t n0 = e2m1_encode(f[16 * b + i] * m), n1 = e2m1_encode(f[16 * b + i + 1] * m);
        if (n0 == 8) n0 = 0;
        if (n1 == 8) n1 = 0;
        vr[(16 * b + i) >> 1] = (uint8_t)(n0 | (n1 << 4));
      }
    }
  }
}

// acc[rows][H] (FP32) += decode of one source; call once per source in rank order, acc starting at +0.
void fp4ar_oracle_decode_acc(float* acc, int rows, const uint8_t* v, long v_stride, const uint8_t* s, long s_stride,
                             const float* rs, float rs_static) {
#pragma omp parallel for
  for (int r = 0; r < rows; r++)
    decode_acc_row(acc + (size_t)r * H, v + (size_t)r * v_stride, s + (size_t)r * s_stride, rs ? rs[r] : rs_static);
}

void fp4ar_oracle_f32_to_bf16(const float* x, uint16_t* out, long n) {
#pragma omp parallel for
  for (long i = 0; i < n; i++) out[i] = f32_to_bf16(x[i]);
}

void fp4ar_oracle_canon_neg0(const uint32_t* in, uint32_t* out, long n) {
  for (long i = 0; i < n; i++) {
    uint32_t w = in[i], r = 0;
    for (int k = 0; k < 8; k++) { uint32_t nib = (w >> (4 * k)) & 15; if (nib == 8) nib = 0; r |= nib << (4 * k); }
    out[i] = r;
  }
}

float fp4ar_oracle_row_sumsq(const float* z) { return row_sumsq(z); }

// ---- the full operator ----
// P sources. input_kind 0: xs[r] = BF16 [rows][H]; 1: xs[r] = NVFP4 rows [rows][3456] (values then scales)
// with static scale gs[r].  algo 0 one-shot, 1 two-shot (sum re-encoded with its own row scale; every
// rank outputs the decode of that re-encoding).  epi 0: out = bf16(sum).  epi 1..3: z = sum + res_in,
// res_out = bf16(z), y = (bf16(z) * rinv) * (wbias + w) with rinv = 1/sqrt(sumsq(z)/H + eps);
// epi 1 -> out = bf16(y); epi 2 -> outq rows of 3456 B NVFP4 (global scale qscale);
// epi 3 -> outq rows of 6336 B MXFP8.  sum_f32 (optional) receives the FP32 value that entered the epilogue.
int fp4ar_oracle_allreduce(int P, int rows, int algo, int input_kind, const void* const* xs, const float* gs,
                           int epi, const uint16_t* res_in, const uint16_t* w, float eps, float wbias, float qscale,
                           uint16_t* out, uint16_t* res_out, uint8_t* outq, float* sum_f32) {
  if (P < 1 || P > 8 || rows < 0 || algo < 0 || algo > 1 || input_kind < 0 || input_kind > 1 || epi < 0 || epi > 3)
    return 1;
  if (epi > 0 && (!res_in || !w || !res_out)) return 2;
  if ((epi == 0 || epi == 1) && !out) return 3;
  if (epi >= 2 && !outq) return 3;
  std::vector<float> wf(H, 0.f);
  if (epi > 0) for (int i = 0; i < H; i++) wf[i] = wbias + bf16_to_f32(w[i]);
#pragma omp parallel for
  for (int r = 0; r < rows; r++) {
    std::vector<float> acc(H, 0.f), f(H);
    std::vector<uint8_t> v(VB), s(SB);
    for (int src = 0; src < P; src++) {
      if (input_kind == 0) {
        const uint16_t* x = (const uint16_t*)xs[src] + (size_t)r * H;
        for (int i = 0; i < H; i++) f[i] = bf16_to_f32(x[i]);
        const float rs = encode_row_dynamic(f.data(), v.data(), s.data(), true);
        decode_acc_row(acc.data(), v.data(), s.data(), rs);
      } else {
        const uint8_t* rec = (const uint8_t*)xs[src] + (size_t)r * (VB + SB);
        decode_acc_row(acc.data(), rec, rec + VB, gs[src]);
      }
    }
    if (algo == 1) {
      const float rs2 = encode_row_dynamic(acc.data(), v.data(), s.data(), true);
      std::fill(acc.begin(), acc.end(), 0.f);
      decode_acc_row(acc.data(), v.data(), s.data(), rs2);
    }
    if (sum_f32) std::memcpy(sum_f32 + (size_t)r * H, acc.data(), H * sizeof(float));
    if (epi == 0) {
      for (int i = 0; i < H; i++) out[(size_t)r * H + i] = f32_to_bf16(acc[i]);
      continue;
    }
    std::vector<float> z(H), yb(H);
    for (int i = 0; i < H; i++) z[i] = acc[i] + bf16_to_f32(res_in[(size_t)r * H + i]);
    const float ss = row_sumsq(z.data());
    const float rinv = 1.0f / std::sqrt(ss / (float)H + eps);
    for (int i = 0; i < H; i++) {
      const uint16_t zb = f32_to_bf16(z[i]);
      res_out[(size_t)r * H + i] = zb;
      const float y = (bf16_to_f32(zb) * rinv) * wf[i];
      const uint16_t yh = f32_to_bf16(y);
      yb[i] = bf16_to_f32(yh);
      if (epi == 1) out[(size_t)r * H + i] = yh;
    }
    if (epi == 2) quant_row_nvfp4_out(yb.data(), qscale, outq + (size_t)r * (VB + SB), outq + (size_t)r * (VB + SB) + VB);
    if (epi == 3) quant_row_mxfp8_out(yb.data(), outq + (size_t)r * (H + PAIRS), outq + (size_t)r * (H + PAIRS) + H);
  }
  return 0;
}

// Stand-alone add + Gemma RMSNorm on a BF16 input (the epilogue above with `x` in place of the sum).
int fp4ar_oracle_add_rmsnorm(int rows, const uint16_t* x, const uint16_t* res_in, const uint16_t* w, float eps,
                             float wbias, int epi, float qscale, uint16_t* out, uint16_t* res_out, uint8_t* outq) {
  if (epi < 1 || epi > 3) return 1;
  std::vector<float> wf(H);
  for (int i = 0; i < H; i++) wf[i] = wbias + bf16_to_f32(w[i]);
#pragma omp parallel for
  for (int r = 0; r < rows; r++) {
    std::vector<float> z(H), yb(H);
    for (int i = 0; i < H; i++) z[i] = bf16_to_f32(x[(size_t)r * H + i]) + bf16_to_f32(res_in[(size_t)r * H + i]);
    const float ss = row_sumsq(z.data());
    const float rinv = 1.0f / std::sqrt(ss / (float)H + eps);
    for (int i = 0; i < H; i++) {
      const uint16_t zb = f32_to_bf16(z[i]);
      res_out[(size_t)r * H + i] = zb;
      const uint16_t yh = f32_to_bf16((bf16_to_f32(zb) * rinv) * wf[i]);
      yb[i] = bf16_to_f32(yh);
      if (epi == 1) out[(size_t)r * H + i] = yh;
    }
    if (epi == 2) quant_row_nvfp4_out(yb.data(), qscale, outq + (size_t)r * (VB + SB), outq + (size_t)r * (VB + SB) + VB);
    if (epi == 3) quant_row_mxfp8_out(yb.data(), outq + (size_t)r * (H + PAIRS), outq + (size_t)r * (H + PAIRS) + H);
  }
  return 0;
}

}  // extern "C"
