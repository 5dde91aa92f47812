// Instantiations of the fused AllReduce kernel: two ranks, one-shot, BF16 input.
#include "ar_table.h"
namespace fp4ar {
void ar_register_p2(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<2, 0, 0, 0, 3>();
  out[(*n)++] = make_entry<2, 0, 0, 1, 3>();
  out[(*n)++] = make_entry<2, 0, 0, 2, 3>();
  out[(*n)++] = make_entry<2, 0, 0, 3, 3>();
}
}  // namespace fp4ar
