// Instantiations of the fused AllReduce kernel: eight ranks, two-shot, NVFP4 and producer-pushed input.
#include "ar_table.h"
namespace fp4ar {
void ar_register_p8b(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<8, 1, 1, 0, 3>();
  out[(*n)++] = make_entry<8, 1, 1, 1, 3>();
  out[(*n)++] = make_entry<8, 1, 1, 2, 3>();
  out[(*n)++] = make_entry<8, 1, 1, 3, 3>();
  out[(*n)++] = make_entry<8, 1, 2, 0, 3>();
  out[(*n)++] = make_entry<8, 1, 2, 1, 3>();
  out[(*n)++] = make_entry<8, 1, 2, 2, 3>();
  out[(*n)++] = make_entry<8, 1, 2, 3, 3>();
}
}  // namespace fp4ar
