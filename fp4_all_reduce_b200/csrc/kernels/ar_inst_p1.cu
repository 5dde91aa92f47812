// Instantiations of the fused AllReduce kernel: single rank (encode, decode of the own encoding, epilogue).
#include "ar_table.h"
namespace fp4ar {
void ar_register_p1(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<1, 0, 0, 0, 3>();
  out[(*n)++] = make_entry<1, 0, 0, 1, 3>();
  out[(*n)++] = make_entry<1, 0, 0, 2, 3>();
  out[(*n)++] = make_entry<1, 0, 0, 3, 3>();
  out[(*n)++] = make_entry<1, 0, 1, 0, 3>();
  out[(*n)++] = make_entry<1, 0, 1, 1, 3>();
  out[(*n)++] = make_entry<1, 0, 1, 2, 3>();
  out[(*n)++] = make_entry<1, 0, 1, 3, 3>();
}
}  // namespace fp4ar
