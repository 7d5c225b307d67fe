// cudeep::kernels matmul launchers: argument checks and dispatch between the
// tcgen05 TF32 GEMM and the strict SIMT GEMMs.
#include "cudeep/kernels/matmul.cuh"

#include "gemm_f16.h"
#include "gemm_simt.h"
#include "gemm_tf32.h"
#include "epilogue_math.cuh"

namespace cudeep {
namespace kernels {

namespace {

void check_dims(const void* a, const void* b, const void* c, int m, int n, int k) {
    CB200_REQUIRE(a != nullptr && b != nullptr && c != nullptr, "matmul: null operand pointer");
    CB200_REQUIRE(m > 0 && n > 0 && k > 0, "matmul: M, N and K must be positive");
}

// Shapes worth a tensor-core tile; below this the strict FP32 kernel is both
// exact and no slower.
bool tensor_core_worthwhile(int m, int n, int k) { return m >= 64 && n >= 64 && k >= 32; }

}  // namespace

template <>
void launch_matmul_kernel<float>(const float* A, const float* B, float* C, int M, int N, int K,
                                 cudaStream_t stream) {
    check_dims(A, B, C, M, N, K);
    if (tensor_core_worthwhile(M, N, K) &&
        cudeep_b200::gemm_tf32_supported(A, B, C, M, N, K, /*b_is_nk=*/false)) {
        cudeep_b200::gemm_tf32(A, B, false, C, M, N, K, nullptr, false, cudeep_b200::EPI_NONE,
                               cudeep_b200::GemmTuning{}, stream);
    } else {
        cudeep_b200::gemm_simt<float>(A, B, false, C, M, N, K, nullptr, false,
                                      cudeep_b200::EPI_NONE, stream);
    }
}

template <>
void launch_matmul_kernel<double>(const double* A, const double* B, double* C, int M, int N, int K,
                                  cudaStream_t stream) {
    check_dims(A, B, C, M, N, K);
    cudeep_b200::gemm_simt<double>(A, B, false, C, M, N, K, nullptr, false, cudeep_b200::EPI_NONE,
                                   stream);
}

template <>
void launch_matmul_kernel_fp32<float>(const float* A, const float* B, float* C, int M, int N, int K,
                                      cudaStream_t stream) {
    check_dims(A, B, C, M, N, K);
    cudeep_b200::gemm_simt<float>(A, B, false, C, M, N, K, nullptr, false, cudeep_b200::EPI_NONE,
                                  stream);
}

template <>
void launch_matmul_kernel_fp32<double>(const double* A, const double* B, double* C, int M, int N,
                                       int K, cudaStream_t stream) {
    launch_matmul_kernel<double>(A, B, C, M, N, K, stream);
}

template <typename T>
void launch_matmul_tiled_kernel(const T* A, const T* B, T* C, int M, int N, int K, int /*tile_size*/,
                                cudaStream_t stream) {
    launch_matmul_kernel<T>(A, B, C, M, N, K, stream);
}
template void launch_matmul_tiled_kernel<float>(const float*, const float*, float*, int, int, int,
                                                int, cudaStream_t);
template void launch_matmul_tiled_kernel<double>(const double*, const double*, double*, int, int,
                                                 int, int, cudaStream_t);

void launch_matmul_kernel_fp16(const __half* A, const __half* B, float* C, int M, int N, int K,
                               cudaStream_t stream) {
    check_dims(A, B, C, M, N, K);
    // Tensor cores (FP16 products are exact, FP32 accumulation) for aligned shapes of at least a
    // tile; the SIMT kernel otherwise.
    if (cudeep_b200::gemm_f16_supported(A, B, M, N, K))
        cudeep_b200::gemm_f16(A, B, C, M, N, K, 0, 0, 0, stream);
    else
        cudeep_b200::gemm_simt_half(A, B, C, M, N, K, stream);
}

void launch_matmul_kernel_bf16(const __nv_bfloat16* A, const __nv_bfloat16* B, float* C, int M, int N, int K,
                               cudaStream_t stream) {
    check_dims(A, B, C, M, N, K);
    if (cudeep_b200::gemm_f16_supported(A, B, M, N, K))
        cudeep_b200::gemm_bf16(A, B, C, M, N, K, 0, stream);
    else
        cudeep_b200::gemm_simt_bf16(A, B, C, M, N, K, stream);
}

void launch_matmul_fused_act(const float* A, const float* B, float* C, int M, int N, int K,
                             GemmEpilogue epilogue, cudaStream_t stream) {
    check_dims(A, B, C, M, N, K);
    const int act = static_cast<int>(epilogue);
    CB200_REQUIRE(act >= 0 && act <= 4, "matmul: unknown epilogue");
    if (tensor_core_worthwhile(M, N, K) &&
        cudeep_b200::gemm_tf32_supported(A, B, C, M, N, K, false)) {
        cudeep_b200::gemm_tf32(A, B, false, C, M, N, K, nullptr, false, act,
                               cudeep_b200::GemmTuning{}, stream);
    } else {
        cudeep_b200::gemm_simt<float>(A, B, false, C, M, N, K, nullptr, false, act, stream);
    }
}

void launch_linear_forward(const float* x, const float* W, const float* bias, float* y, int M,
                           int N, int K, GemmEpilogue epilogue, cudaStream_t stream) {
    check_dims(x, W, y, M, N, K);
    const int act = static_cast<int>(epilogue);
    CB200_REQUIRE(act >= 0 && act <= 4, "linear: unknown epilogue");
    if (tensor_core_worthwhile(M, N, K) &&
        cudeep_b200::gemm_tf32_supported(x, W, y, M, N, K, /*b_is_nk=*/true)) {
        cudeep_b200::gemm_tf32(x, W, true, y, M, N, K, bias, false, act, cudeep_b200::GemmTuning{},
                               stream);
    } else {
        cudeep_b200::gemm_simt<float>(x, W, true, y, M, N, K, bias, false, act, stream);
    }
}

void launch_matmul_tn(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t stream) {
    check_dims(A, B, C, M, N, K);
    if (tensor_core_worthwhile(M, N, K) && cudeep_b200::gemm_tf32_tn_supported(A, B, M, N, K)) {
        cudeep_b200::gemm_tf32_tn(A, B, C, M, N, K, cudeep_b200::GemmTuning{}, stream);
    } else {
        cudeep_b200::gemm_simt_tn(A, B, C, M, N, K, stream);
    }
}

void launch_matmul_nt(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t stream) {
    launch_linear_forward(A, B, nullptr, C, M, N, K, GemmEpilogue::None, stream);
}

void launch_linear_forward(const double* x, const double* W, const double* bias, double* y, int M,
                           int N, int K, GemmEpilogue epilogue, cudaStream_t stream) {
    check_dims(x, W, y, M, N, K);
    cudeep_b200::gemm_simt<double>(x, W, true, y, M, N, K, bias, false, static_cast<int>(epilogue),
                                   stream);
}

}  // namespace kernels
}  // namespace cudeep
