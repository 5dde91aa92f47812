// Experimental variant 1 of the fused AllReduce kernel for the two-shot shapes that are bound by latency inside the
// SM: the slow halves of the window polls are out-of-line calls (FP4AR_COLD_PATHS), which shrinks the kernel bodies.
// Same arithmetic, same protocol, same results; selected with FP4AR_KERNEL_VARIANT=1 in the environment (or bits 8-15
// of tune[1]); the product kernels are untouched by this file.
#define FP4AR_KERNEL_NAME ar_kernel_cold
#define FP4AR_KERNEL_VARIANT_ID 1
#define FP4AR_COLD_PATHS 1
#include "ar_table.h"
namespace fp4ar {
void ar_register_cold(ArKernelEntry* out, int* n) {
  out[(*n)++] = make_entry<4, 1, 0, 0, 3>();
  out[(*n)++] = make_entry<4, 1, 0, 1, 3>();
  out[(*n)++] = make_entry<4, 1, 1, 0, 3>();
  out[(*n)++] = make_entry<4, 1, 1, 1, 3>();
  out[(*n)++] = make_entry<4, 1, 2, 1, 3>();
  out[(*n)++] = make_entry<8, 1, 0, 0, 3>();
  out[(*n)++] = make_entry<8, 1, 0, 1, 3>();
  out[(*n)++] = make_entry<8, 1, 1, 0, 3>();
  out[(*n)++] = make_entry<8, 1, 1, 1, 3>();
  out[(*n)++] = make_entry<8, 1, 2, 1, 3>();
}
}  // namespace fp4ar
