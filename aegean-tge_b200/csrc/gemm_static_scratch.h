// Declaration of the product entry point that needs no allocated scratch.
//
// This entry point has no counterpart in the reference engine; it exists for
// embedders of this library.  See gemm_static_scratch.cu for the contract.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch buffer, in float32 elements (16 MiB per GPU that loads the library).
#define TGE_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

// out = x . w^T (+ epilogue), bfloat16 operands, like tge_gemm_tcgen05, with the k-split partial
// sums kept in a buffer that is part of the library image instead of one the caller allocates.
// Returns the number of kernels launched, TGE_UNSUPPORTED (-100) for shapes TMA cannot address,
// or a negative code with a message in tge_last_error().
int tge_gemm_tcgen05_static_scratch(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                    void* out, long long ldo, int M, int N, int K, int epilogue, int* status,
                                    cudaStream_t stream);

#ifdef __cplusplus
}
#endif
