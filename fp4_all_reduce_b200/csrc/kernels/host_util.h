// Small host-side helpers shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>
#include "../include/fp4ar.h"

namespace fp4ar {

constexpr int kMaxRanksOps = FP4AR_MAX_RANKS;

// Remembers the text of the last failed CUDA call for fp4ar_last_cuda_error().
void set_last_cuda_error(cudaError_t e, const char* where);
int cuda_fail();                 // records cudaGetLastError(), returns FP4AR_ERR_CUDA
int cuda_check_launch();         // FP4AR_OK, or FP4AR_ERR_CUDA if the launch was rejected
int device_sm_count();           // multiprocessors of the current device (cached per device)

}  // namespace fp4ar
