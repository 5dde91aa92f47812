// Six-warp teams (one pair of a row per lane) for the two-shot algorithm at 8 ranks: BF16 input, every epilogue.
#include "ar_table.h"
namespace fp4ar {
void ar_register_t6p8(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<8, 1, 0, 0, 6>();
  out[(*n)++] = make_entry<8, 1, 0, 1, 6>();
  out[(*n)++] = make_entry<8, 1, 0, 2, 6>();
  out[(*n)++] = make_entry<8, 1, 0, 3, 6>();
}
}  // namespace fp4ar
