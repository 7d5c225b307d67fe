// C++ launchers of the dense-contraction path, Blackwell (sm_100a) build.
//
// The first six declarations keep the names, argument lists and mangled
// symbols of the reference's include/cudeep/kernels/matmul.cuh:8-44, so code
// compiled against that header links against this library unchanged.  All
// matrices are row-major and contiguous; launches are asynchronous on `stream`
// (nullptr = the legacy default stream); errors are std::runtime_error.
//
// Dispatch of the float launcher, launch_matmul_kernel<float>:
//   * tcgen05 TF32 tensor-core GEMM (FP32 accumulate) when M >= 64, N >= 64,
//     K >= 32, K % 4 == 0, N % 4 == 0 and A, B are 16-byte aligned;
//   * strict FP32 SIMT GEMM otherwise, so tiny and odd-shaped products are
//     exact to FP32 rounding.
// launch_matmul_kernel_fp32 is always strict FP32; the double instantiations
// are FP64 SIMT.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace cudeep {
namespace kernels {

// Activation fused into a GEMM epilogue.  GELU is the tanh form.
enum class GemmEpilogue { None, ReLU, GELU, SiLU, Sigmoid };

// ---- reference-compatible surface ------------------------------------------------------

// C[M,N] = A[M,K] * B[K,N].  T = float: TF32 tensor cores for large aligned
// shapes (see above).  T = double: FP64.           (reference matmul.cuh:8-12)
template <typename T>
void launch_matmul_kernel(const T* A, const T* B, T* C, int M, int N, int K,
                          cudaStream_t stream = nullptr);

// Same product in strict element precision.        (reference matmul.cuh:14-18)
template <typename T>
void launch_matmul_kernel_fp32(const T* A, const T* B, T* C, int M, int N, int K,
                               cudaStream_t stream = nullptr);

// Alias of launch_matmul_kernel; `tile_size` is accepted and ignored, as in
// the reference (matmul.cuh:20-25, matmul_kernel.cu:1871-1875).
template <typename T>
void launch_matmul_tiled_kernel(const T* A, const T* B, T* C, int M, int N, int K, int tile_size,
                                cudaStream_t stream = nullptr);

// Half inputs, float output.                        (reference matmul.cuh:27-30)
void launch_matmul_kernel_fp16(const __half* A, const __half* B, float* C, int M, int N, int K,
                               cudaStream_t stream = nullptr);

// C = act(A * B), activation applied in the GEMM epilogue.  (reference matmul.cuh:40-44)
void launch_matmul_fused_act(const float* A, const float* B, float* C, int M, int N, int K,
                             GemmEpilogue epilogue, cudaStream_t stream = nullptr);

// ---- additions ------------------------------------------------------------------------

// BF16 inputs, float output: launch_matmul_kernel_fp16's sibling (the reference has FP16 only).
// Tensor cores (kind::f16 with BF16 operand format) for aligned shapes of at least a tile, the
// SIMT kernel otherwise; products of BF16 values are exact, accumulation is FP32.
void launch_matmul_kernel_bf16(const __nv_bfloat16* A, const __nv_bfloat16* B, float* C, int M, int N, int K,
                               cudaStream_t stream = nullptr);

// y[M,N] = act(x[M,K] * W[N,K]^T + bias[N]) in one kernel.  W is consumed as
// nn.Linear stores it ([out_features, in_features] row-major); bias may be
// nullptr.  Replaces the transpose-copy + GEMM + broadcast_add + activation
// sequence of the reference's nn.Linear.forward (python/cuDeep/nn.py:110-115).
void launch_linear_forward(const float* x, const float* W, const float* bias, float* y, int M,
                           int N, int K, GemmEpilogue epilogue, cudaStream_t stream = nullptr);
void launch_linear_forward(const double* x, const double* W, const double* bias, double* y, int M,
                           int N, int K, GemmEpilogue epilogue, cudaStream_t stream = nullptr);

// The two products of matmul's backward pass without transposed copies (the reference
// materialises b^T and a^T first, python/cuDeep/tensor.py:430-443):
//   launch_matmul_nt: C[M,N] = A[M,K] * B[N,K]^T     (grad_a = grad * b^T)
//   launch_matmul_tn: C[M,N] = A[K,M]^T * B[K,N]     (grad_b = a^T * grad)
// Same precision rule as launch_matmul_kernel<float>.
void launch_matmul_nt(const float* A, const float* B, float* C, int M, int N, int K,
                      cudaStream_t stream = nullptr);
void launch_matmul_tn(const float* A, const float* B, float* C, int M, int N, int K,
                      cudaStream_t stream = nullptr);

}  // namespace kernels
}  // namespace cudeep
