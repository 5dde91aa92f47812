// Six-warp teams (one pair of a row per lane) for the two-shot algorithm at 4 ranks: NVFP4 and producer-pushed input, every epilogue.
#include "ar_table.h"
namespace fp4ar {
void ar_register_t6p4b(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<4, 1, 1, 0, 6>();
  out[(*n)++] = make_entry<4, 1, 1, 1, 6>();
  out[(*n)++] = make_entry<4, 1, 1, 2, 6>();
  out[(*n)++] = make_entry<4, 1, 1, 3, 6>();
  out[(*n)++] = make_entry<4, 1, 2, 0, 6>();
  out[(*n)++] = make_entry<4, 1, 2, 1, 6>();
  out[(*n)++] = make_entry<4, 1, 2, 2, 6>();
  out[(*n)++] = make_entry<4, 1, 2, 3, 6>();
}
}  // namespace fp4ar
