// Instantiations of the fused AllReduce kernel: the losing algorithm of each degree, kept for comparison (two-shot at 2 ranks, one-shot at 4 and 8).
#include "ar_table.h"
namespace fp4ar {
void ar_register_cmp(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<2, 1, 0, 0, 3>();
  out[(*n)++] = make_entry<2, 1, 1, 0, 3>();
  out[(*n)++] = make_entry<4, 0, 0, 0, 3>();
  out[(*n)++] = make_entry<4, 0, 1, 0, 3>();
  out[(*n)++] = make_entry<8, 0, 0, 0, 3>();
  out[(*n)++] = make_entry<8, 0, 1, 0, 3>();
}
}  // namespace fp4ar
