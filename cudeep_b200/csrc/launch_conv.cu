// cudeep::kernels conv2d forward launchers: dispatch between the implicit-GEMM
// tensor-core path and the direct strict-precision kernel.
#include "cudeep/kernels/conv.cuh"

#include "conv_igemm.h"
#include "epilogue_math.cuh"

namespace cudeep {
namespace kernels {

namespace {
cudeep_b200::ConvShape make_shape(int batch, int in_c, int out_c, int in_h, int in_w, int k_h, int k_w,
                                  int s_h, int s_w, int p_h, int p_w) {
    return cudeep_b200::ConvShape{batch, in_c, out_c, in_h, in_w, k_h, k_w, s_h, s_w, p_h, p_w};
}
}  // namespace

void launch_conv2d_forward_fused(const float* input, const float* weight, const float* bias,
                                 float* output, int batch, int in_channels, int out_channels,
                                 int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                 int stride_w, int pad_h, int pad_w, GemmEpilogue epilogue,
                                 cudaStream_t stream) {
    CB200_REQUIRE(input != nullptr && weight != nullptr && output != nullptr,
                  "conv2d: null tensor pointer");
    const int act = static_cast<int>(epilogue);
    CB200_REQUIRE(act >= 0 && act <= 4, "conv2d: unknown epilogue");
    const cudeep_b200::ConvShape s = make_shape(batch, in_channels, out_channels, in_h, in_w, kernel_h,
                                                kernel_w, stride_h, stride_w, pad_h, pad_w);
    cudeep_b200::check_conv_shape(s);
    if (cudeep_b200::conv2d_igemm_supported(s))
        cudeep_b200::conv2d_igemm(input, weight, bias, output, s, act, stream);
    else
        cudeep_b200::conv2d_direct<float>(input, weight, bias, output, s, act, stream);
}

void launch_conv2d_forward_fused_layout(const float* input, Layout input_layout, const float* weight,
                                        const float* bias, float* output, int batch, int in_channels,
                                        int out_channels, int in_h, int in_w, int kernel_h, int kernel_w,
                                        int stride_h, int stride_w, int pad_h, int pad_w, GemmEpilogue epilogue,
                                        cudaStream_t stream) {
    if (input_layout == Layout::NCHW) {
        launch_conv2d_forward_fused(input, weight, bias, output, batch, in_channels, out_channels, in_h, in_w,
                                    kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, epilogue, stream);
        return;
    }
    CB200_REQUIRE(input_layout == Layout::NHWC, "conv2d: unknown input layout");
    CB200_REQUIRE(input != nullptr && weight != nullptr && output != nullptr, "conv2d: null tensor pointer");
    const int act = static_cast<int>(epilogue);
    CB200_REQUIRE(act >= 0 && act <= 4, "conv2d: unknown epilogue");
    const cudeep_b200::ConvShape s = make_shape(batch, in_channels, out_channels, in_h, in_w, kernel_h,
                                                kernel_w, stride_h, stride_w, pad_h, pad_w);
    cudeep_b200::check_conv_shape(s);
    CB200_REQUIRE(cudeep_b200::conv2d_igemm_takes_nhwc_input(input, s),
                  "conv2d: an NHWC input needs C % 4 == 0, a 16-byte aligned pointer and a shape the tensor-core "
                  "path takes (OC >= 32, at least 64 output pixels, strides 1..8, padding smaller than the filter, "
                  "more channels than a row-packed first layer)");
    cudeep_b200::conv2d_igemm(input, weight, bias, output, s, act, stream, false, nullptr, /*input_is_nhwc=*/true);
}

template <>
void launch_conv2d_forward_kernel<float>(const float* input, const float* weight, const float* bias,
                                         float* output, int batch, int in_channels, int out_channels,
                                         int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                         int stride_w, int pad_h, int pad_w, cudaStream_t stream) {
    launch_conv2d_forward_fused(input, weight, bias, output, batch, in_channels, out_channels, in_h,
                                in_w, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
                                GemmEpilogue::None, stream);
}

template <>
void launch_conv2d_forward_kernel<double>(const double* input, const double* weight,
                                          const double* bias, double* output, int batch,
                                          int in_channels, int out_channels, int in_h, int in_w,
                                          int kernel_h, int kernel_w, int stride_h, int stride_w,
                                          int pad_h, int pad_w, cudaStream_t stream) {
    CB200_REQUIRE(input != nullptr && weight != nullptr && output != nullptr,
                  "conv2d: null tensor pointer");
    const cudeep_b200::ConvShape s = make_shape(batch, in_channels, out_channels, in_h, in_w, kernel_h,
                                                kernel_w, stride_h, stride_w, pad_h, pad_w);
    cudeep_b200::conv2d_direct<double>(input, weight, bias, output, s, cudeep_b200::EPI_NONE, stream);
}

}  // namespace kernels
}  // namespace cudeep
