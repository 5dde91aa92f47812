// Table of compiled fused-kernel shapes.  Each ar_inst_*.cu translation unit instantiates a slice of
// the (P, algorithm, input, epilogue) space and registers it here; the runtime looks shapes up by key.
#pragma once
#include "ar_kernel.cuh"

namespace fp4ar {

struct ArKernelEntry {
  int P, algo, input, epi, T;
  const void* fn;
  int team_bytes, cta_extra, max_teams;
  int variant;      // 0 = the product kernel; other values are experimental builds of the same template
};

#ifndef FP4AR_KERNEL_VARIANT_ID
#define FP4AR_KERNEL_VARIANT_ID 0
#endif

constexpr int kDefaultTeamWarps = 3;   // warps per row team unless a launch asks for another compiled width

// Internal linkage on purpose: experimental translation units instantiate this template for shapes that a product unit
// also instantiates, with a different kernel behind it; every unit must keep its own copy.
template <int P, int ALGO, int IN, int EPI, int T>
static inline ArKernelEntry make_entry() {
  using S = ArShape<P, ALGO, IN, EPI, T>;
  ArKernelEntry e;
  e.P = P; e.algo = ALGO; e.input = IN; e.epi = EPI; e.T = T;
  e.fn = reinterpret_cast<const void*>(&FP4AR_KERNEL_NAME<P, ALGO, IN, EPI, T>);
  e.team_bytes = S::kTeamBytes; e.cta_extra = S::kCtaExtra; e.max_teams = S::kMaxTeams;
  e.variant = FP4AR_KERNEL_VARIANT_ID;
  return e;
}

// Defined once per instantiation unit; each appends its entries.
void ar_register_p1(ArKernelEntry* out, int* n);
void ar_register_p2(ArKernelEntry* out, int* n);
void ar_register_p2b(ArKernelEntry* out, int* n);
void ar_register_p4(ArKernelEntry* out, int* n);
void ar_register_p4b(ArKernelEntry* out, int* n);
void ar_register_p8(ArKernelEntry* out, int* n);
void ar_register_p8b(ArKernelEntry* out, int* n);
void ar_register_cmp(ArKernelEntry* out, int* n);
void ar_register_t6(ArKernelEntry* out, int* n);     // six-warp teams, two-shot shapes of 4 and 8 ranks (ar_inst_t6.cu)
void ar_register_t6x4(ArKernelEntry* out, int* n);   // variant 2: six-warp teams, four teams per CTA (ar_inst_t6x4.cu)
void ar_register_cold(ArKernelEntry* out, int* n);   // variant 1: slow poll paths out of line (ar_inst_cold.cu)

}  // namespace fp4ar
