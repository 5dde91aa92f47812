// Experimental variant 2 of the fused AllReduce kernel: six-warp teams with FOUR teams per CTA (24 warps per SM at
// 80 registers, some spilling) for the two-shot shapes of 4 and 8 ranks.  Selected with FP4AR_KERNEL_VARIANT=2 (or
// bits 8-15 of tune[1]) together with tune[2] = 6; the product kernels are untouched by this file.
#define FP4AR_KERNEL_NAME ar_kernel_t6x4
#define FP4AR_KERNEL_VARIANT_ID 2
#define FP4AR_T6_TEAMS 4
#include "ar_table.h"
namespace fp4ar {
void ar_register_t6x4(ArKernelEntry* out, int* n) {
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
