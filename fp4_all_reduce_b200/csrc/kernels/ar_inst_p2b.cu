// Instantiations of the fused AllReduce kernel: two ranks, one-shot, NVFP4 and producer-pushed input.
#include "ar_table.h"
namespace fp4ar {
void ar_register_p2b(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<2, 0, 1, 0, 3>();
  out[(*n)++] = make_entry<2, 0, 1, 1, 3>();
  out[(*n)++] = make_entry<2, 0, 1, 2, 3>();
  out[(*n)++] = make_entry<2, 0, 1, 3, 3>();
  out[(*n)++] = make_entry<2, 0, 2, 0, 3>();
  out[(*n)++] = make_entry<2, 0, 2, 1, 3>();
  out[(*n)++] = make_entry<2, 0, 2, 2, 3>();
  out[(*n)++] = make_entry<2, 0, 2, 3, 3>();
}
}  // namespace fp4ar
