// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// extern "C" doorway to the reference's own launchers, compiled together with
// the reference's unmodified sources (see oracle/Makefile, target `ref`) into
// oracle/_ref/libcudeep_ref.so.  It lets tests and bench.py run the reference's
// CUDA kernels on the same device and inputs as this library.  Exceptions the
// reference throws are turned into a non-zero return code.
#include "cudeep/kernels/matmul.cuh"
#include "cudeep/kernels/conv.cuh"

#include <cstdio>
#include <exception>

namespace {
template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "cudeep reference: %s\n", e.what());
    } catch (...) {
        std::fprintf(stderr, "cudeep reference: unknown exception\n");
    }
    return 1;
}
}  // namespace

extern "C" {

int cudeep_ref_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K, void* stream) {
    return guarded([&] {
        cudeep::kernels::launch_matmul_kernel<float>(A, B, C, M, N, K, static_cast<cudaStream_t>(stream));
    });
}

int cudeep_ref_matmul_f32_strict(const float* A, const float* B, float* C, int M, int N, int K, void* stream) {
    return guarded([&] {
        cudeep::kernels::launch_matmul_kernel_fp32<float>(A, B, C, M, N, K, static_cast<cudaStream_t>(stream));
    });
}

int cudeep_ref_matmul_fused_act(const float* A, const float* B, float* C, int M, int N, int K, int epilogue,
                                void* stream) {
    return guarded([&] {
        cudeep::kernels::launch_matmul_fused_act(A, B, C, M, N, K,
                                                 static_cast<cudeep::kernels::GemmEpilogue>(epilogue),
                                                 static_cast<cudaStream_t>(stream));
    });
}

int cudeep_ref_conv2d_forward_f32(const float* input, const float* weight, const float* bias, float* output,
                                  int batch, int in_c, int out_c, int in_h, int in_w, int k_h, int k_w,
                                  int s_h, int s_w, int p_h, int p_w, void* stream) {
    return guarded([&] {
        cudeep::kernels::launch_conv2d_forward_kernel<float>(input, weight, bias, output, batch, in_c, out_c,
                                                             in_h, in_w, k_h, k_w, s_h, s_w, p_h, p_w,
                                                             static_cast<cudaStream_t>(stream));
    });
}

}  // extern "C"
