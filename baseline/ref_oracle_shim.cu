// Host-side bridge to the reference project's own CPU oracle (`namespace cpu` of bench/codec/codec_bench.cu:594-674),
// so that the host model of this repository can be compared with it on a machine without a GPU.
//
// The reference file is included untouched (its `main` is renamed by the preprocessor and never called; its kernels
// are compiled but never launched).  Only host functions of `cpu::` run: init, enc_slot, oneshot, twoshot.
#define main fp4ar_reference_codec_bench_main
#include "bench/codec/codec_bench.cu"
#undef main

// xs: P pointers to [R][6144] BF16 bit patterns; out: [R][6144] BF16 bit patterns.
extern "C" int ref_cpu_allreduce(int P, int R, const uint16_t* const* xs, int two_shot, uint16_t* out) {
  if (P < 1 || P > 8 || R < 1 || !xs || !out) return 1;
  static bool inited = false;
  if (!inited) { cpu::init(); inited = true; }
  std::vector<std::vector<uint8_t>> slots(P);
  for (int s = 0; s < P; s++) {
    std::vector<uint16_t> x(xs[s], xs[s] + (size_t)R * H);
    cpu::enc_slot(x, R, slots[s], true);
  }
  std::vector<uint16_t> o;
  if (two_shot) cpu::twoshot(slots.data(), P, R, o); else cpu::oneshot(slots.data(), P, R, o);
  memcpy(out, o.data(), (size_t)R * H * 2);
  return 0;
}

// One row: values [3072], scales [384], row scale, as cpu::enc_row writes them.
extern "C" int ref_cpu_encode_rows(int R, const uint16_t* x, uint8_t* values, uint8_t* scales, float* rs, int canon) {
  static bool inited = false;
  if (!inited) { cpu::init(); inited = true; }
  for (int r = 0; r < R; r++) {
    std::vector<float> f(H);
    for (int i = 0; i < H; i++) f[i] = cpu::bf(x[(size_t)r * H + i]);
    cpu::enc_row(f.data(), values + (size_t)r * VB, scales + (size_t)r * SB, rs + r, canon != 0);
  }
  return 0;
}
