// Host entry of the tcgen05 FP16 GEMM (see gemm_f16.cu).
#pragma once

#include "runtime.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace cudeep_b200 {

// True when the tensor-core path takes this problem: sm_100 device, 16-byte aligned A and B,
// K and N multiples of 8 (rows of A[M,K] and B[K,N] are 16-byte multiples), and at least one
// 128 x 64 tile's worth of work.
bool gemm_f16_supported(const void* a, const void* b, int m, int n, int k);

// C[M,N] (FP32) = A[M,K] * B[K,N], FP16 operands multiplied exactly, FP32 accumulation.
// ctas: 0 = choose, 1 or 2 CTAs per MMA.  b_lbo / b_sbo: 0, or overrides of the B shared-memory
// descriptor offsets (bring-up aid).  Asynchronous on `stream`.
void gemm_f16(const __half* a, const __half* b, float* c, int m, int n, int k, int ctas, uint32_t b_lbo,
              uint32_t b_sbo, cudaStream_t stream);

// The same with BF16 operands (products of BF16 values are exact in FP32 too); the mainloop differs
// from the FP16 one in the operand-format bits of the MMA's instruction descriptor only.
void gemm_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, float* c, int m, int n, int k, int ctas,
               cudaStream_t stream);

}  // namespace cudeep_b200
