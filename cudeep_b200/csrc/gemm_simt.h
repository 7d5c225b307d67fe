// Strict-precision SIMT GEMMs (FP32 FFMA and FP64 DFMA), any shape.
#pragma once

#include "runtime.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace cudeep_b200 {

// C[M,N] = act(A[M,K] * B + bias) with IEEE fused multiply-adds in the element type.
//   b_is_nk == false: B is [K,N] row-major;  true: B is [N,K] row-major.
//   bias: nullptr, N values (per column) or M values (bias_per_row).
template <typename T>
void gemm_simt(const T* a, const T* b, bool b_is_nk, T* c, int m, int n, int k, const T* bias,
               bool bias_per_row, int act, cudaStream_t stream);

// C[M,N] = A^T * B with A stored [K,M], B stored [K,N]; strict FP32.
void gemm_simt_tn(const float* a, const float* b, float* c, int m, int n, int k, cudaStream_t stream);

// C[M,N] = A[M,K] * B[K,N] with half inputs widened to FP32 and FP32 accumulation.
void gemm_simt_half(const __half* a, const __half* b, float* c, int m, int n, int k,
                    cudaStream_t stream);
void gemm_simt_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, float* c, int m, int n, int k,
                    cudaStream_t stream);

}  // namespace cudeep_b200
