// Instantiations of the fused AllReduce kernel with six-warp teams (one 32-value pair per lane and row, three teams
// per CTA = 18 warps) for the headline shapes of every degree: more warps per SM and a shorter critical path per row
// at the price of six-warp team barriers.  Selected with tune[2] = 6 (bench_cli --team-warps 6); not a default.
#include "ar_table.h"
namespace fp4ar {
void ar_register_t6(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<1, 0, 0, 0, 6>();
  out[(*n)++] = make_entry<1, 0, 0, 1, 6>();
  out[(*n)++] = make_entry<1, 0, 1, 0, 6>();
  out[(*n)++] = make_entry<1, 0, 1, 1, 6>();
  out[(*n)++] = make_entry<2, 0, 0, 0, 6>();
  out[(*n)++] = make_entry<2, 0, 0, 1, 6>();
  out[(*n)++] = make_entry<2, 0, 1, 0, 6>();
  out[(*n)++] = make_entry<2, 0, 1, 1, 6>();
  out[(*n)++] = make_entry<2, 0, 2, 1, 6>();
  out[(*n)++] = make_entry<4, 1, 0, 0, 6>();
  out[(*n)++] = make_entry<4, 1, 0, 1, 6>();
  out[(*n)++] = make_entry<4, 1, 1, 0, 6>();
  out[(*n)++] = make_entry<4, 1, 1, 1, 6>();
  out[(*n)++] = make_entry<4, 1, 2, 1, 6>();
  out[(*n)++] = make_entry<8, 1, 0, 0, 6>();
  out[(*n)++] = make_entry<8, 1, 0, 1, 6>();
  out[(*n)++] = make_entry<8, 1, 1, 0, 6>();
  out[(*n)++] = make_entry<8, 1, 1, 1, 6>();
  out[(*n)++] = make_entry<8, 1, 2, 1, 6>();
}
}  // namespace fp4ar
