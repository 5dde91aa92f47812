// Instantiations of the fused AllReduce kernel: eight ranks, two-shot, BF16 input.
#include "ar_table.h"
namespace fp4ar {
void ar_register_p8(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<8, 1, 0, 0, 3>();
  out[(*n)++] = make_entry<8, 1, 0, 1, 3>();
  out[(*n)++] = make_entry<8, 1, 0, 2, 3>();
  out[(*n)++] = make_entry<8, 1, 0, 3, 3>();
}
}  // namespace fp4ar
