// Table of compiled fused-kernel shapes.  Each ar_inst_*.cu translation unit instantiates a slice of
// the (P, algorithm, input, epilogue) space and registers it here; the runtime looks shapes up by key.
#pragma once
#include "ar_kernel.cuh"

namespace fp4ar {

struct ArKernelEntry {
  int P, algo, input, epi, T;
  const void* fn;
  int team_bytes, cta_extra, max_teams;
};

// Warps per row team unless a launch asks for another compiled width: six for the two-shot algorithm at four and
// eight ranks (one pair per lane: the shortest chain per step, 18 warps per SM), three everywhere else.
constexpr int kDefaultTeamWarps = 3;
inline int default_team_warps(int nranks, int algo) { return (algo == 1 && nranks >= 4) ? 6 : kDefaultTeamWarps; }

// Internal linkage on purpose: experimental translation units instantiate this template for shapes that a product unit
// also instantiates, with a different kernel behind it; every unit must keep its own copy.
template <int P, int ALGO, int IN, int EPI, int T>
static inline ArKernelEntry make_entry() {
  using S = ArShape<P, ALGO, IN, EPI, T>;
  ArKernelEntry e;
  e.P = P; e.algo = ALGO; e.input = IN; e.epi = EPI; e.T = T;
  e.fn = reinterpret_cast<const void*>(&ar_kernel<P, ALGO, IN, EPI, T>);
  e.team_bytes = S::kTeamBytes; e.cta_extra = S::kCtaExtra; e.max_teams = S::kMaxTeams;
  return e;
}

// Defined once per instantiation unit; each appends its entries.
void ar_register_p1(ArKernelEntry* out, int* n);      // one rank
void ar_register_p2(ArKernelEntry* out, int* n);      // two ranks, one-shot, BF16 input
void ar_register_p2b(ArKernelEntry* out, int* n);     // two ranks, one-shot, NVFP4 / pushed input
void ar_register_p4(ArKernelEntry* out, int* n);      // four ranks, two-shot, three-warp teams
void ar_register_p4b(ArKernelEntry* out, int* n);
void ar_register_p8(ArKernelEntry* out, int* n);      // eight ranks, two-shot, three-warp teams
void ar_register_p8b(ArKernelEntry* out, int* n);
void ar_register_cmp(ArKernelEntry* out, int* n);     // the other algorithm of each degree (two-shot at 2, one-shot at 4 and 8)
void ar_register_t6p4(ArKernelEntry* out, int* n);    // four ranks, two-shot, six-warp teams (the default width there)
void ar_register_t6p4b(ArKernelEntry* out, int* n);
void ar_register_t6p8(ArKernelEntry* out, int* n);    // eight ranks, two-shot, six-warp teams
void ar_register_t6p8b(ArKernelEntry* out, int* n);

}  // namespace fp4ar
