// Conv2d backward launchers (reference include/cudeep/kernels/conv.cuh:18-36,
// src/kernels/conv_kernel.cu:337-545).
//
// grad_input: for stride 1 it is itself a convolution - of grad_output with the filters
// flipped in both spatial directions and with their channel axes swapped, padded by
// (KH-1-pad_h, KW-1-pad_w) - so it runs on the forward implicit-GEMM path, whose filter
// packing reads the filters in that order.  The reference instead forms weight^T x grad_output as one big
// GEMM into a [C*KH*KW, N*OH*OW] temporary and scatters it back with col2im.  A strided
// convolution splits its input pixels into stride_h * stride_w parity classes, each the stride-1
// convolution of grad_output with the sub-filter of the taps that reach it (conv_igemm.cu); shapes
// that form does not take use the same path with zeros inserted between the pixels of grad_output.
// FP64 and shapes the tensor-core path does not take use a direct gather kernel.
//
// grad_weight: an implicit GEMM over output pixels on the tensor cores (any stride up to 8)
// (conv_wgrad.cu); otherwise a direct strict-precision kernel (one thread per filter element,
// summing over images and output pixels in a fixed order).
#include "cudeep/kernels/conv.cuh"

#include "conv_igemm.h"
#include "epilogue_math.cuh"

namespace cudeep_b200 {
namespace {

template <typename T>
__global__ void conv2d_backward_data_direct_kernel(const T* __restrict__ dy, const T* __restrict__ w,
                                                   T* __restrict__ dx, ConvShape s, int oh_n, int ow_n,
                                                   long long total) {
    for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int iw = static_cast<int>(idx % s.in_w);
        long long r = idx / s.in_w;
        const int ih = static_cast<int>(r % s.in_h);
        r /= s.in_h;
        const int c = static_cast<int>(r % s.in_c);
        const int n = static_cast<int>(r / s.in_c);
        T acc = T(0);
        for (int oc = 0; oc < s.out_c; ++oc) {
            const T* dyp = dy + (static_cast<long long>(n) * s.out_c + oc) * oh_n * ow_n;
            const T* wp = w + (static_cast<long long>(oc) * s.in_c + c) * s.k_h * s.k_w;
            for (int kh = 0; kh < s.k_h; ++kh) {
                const int oh_num = ih + s.p_h - kh;
                if (oh_num < 0 || oh_num % s.s_h != 0) continue;
                const int oh = oh_num / s.s_h;
                if (oh >= oh_n) continue;
                for (int kw = 0; kw < s.k_w; ++kw) {
                    const int ow_num = iw + s.p_w - kw;
                    if (ow_num < 0 || ow_num % s.s_w != 0) continue;
                    const int ow = ow_num / s.s_w;
                    if (ow >= ow_n) continue;
                    acc += dyp[oh * ow_n + ow] * wp[kh * s.k_w + kw];
                }
            }
        }
        dx[idx] = acc;
    }
}

template <typename T>
__global__ void conv2d_backward_weight_direct_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                     T* __restrict__ dw, ConvShape s, int oh_n, int ow_n,
                                                     long long total) {
    for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int kw = static_cast<int>(idx % s.k_w);
        long long r = idx / s.k_w;
        const int kh = static_cast<int>(r % s.k_h);
        r /= s.k_h;
        const int c = static_cast<int>(r % s.in_c);
        const int oc = static_cast<int>(r / s.in_c);
        T acc = T(0);
        for (int n = 0; n < s.batch; ++n) {
            const T* dyp = dy + (static_cast<long long>(n) * s.out_c + oc) * oh_n * ow_n;
            const T* xp = x + (static_cast<long long>(n) * s.in_c + c) * s.in_h * s.in_w;
            for (int oh = 0; oh < oh_n; ++oh) {
                const int ih = oh * s.s_h - s.p_h + kh;
                if (ih < 0 || ih >= s.in_h) continue;
                for (int ow = 0; ow < ow_n; ++ow) {
                    const int iw = ow * s.s_w - s.p_w + kw;
                    if (iw < 0 || iw >= s.in_w) continue;
                    acc += dyp[oh * ow_n + ow] * xp[ih * s.in_w + iw];
                }
            }
        }
        dw[idx] = acc;
    }
}

unsigned grid_for(long long total) {
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(device_info().num_sms) * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

template <typename T>
void backward_data_direct(const T* dy, const T* w, T* dx, const ConvShape& s, cudaStream_t stream) {
    const long long total = static_cast<long long>(s.batch) * s.in_c * s.in_h * s.in_w;
    CB200_TRACE("conv2d grad_input direct strict %s: N=%d C=%d %dx%d OC=%d, %dx%d stride %dx%d",
                sizeof(T) == 8 ? "FP64" : "FP32", s.batch, s.in_c, s.in_h, s.in_w, s.out_c, s.k_h, s.k_w, s.s_h, s.s_w);
    conv2d_backward_data_direct_kernel<T><<<grid_for(total), 256, 0, stream>>>(dy, w, dx, s, s.out_h(),
                                                                               s.out_w(), total);
    CB200_CHECK_LAUNCH();
}

}  // namespace
}  // namespace cudeep_b200

namespace cudeep {
namespace kernels {

using cudeep_b200::ConvShape;

template <>
void launch_conv2d_backward_data_kernel<float>(const float* grad_output, const float* weight,
                                               float* grad_input, int batch, int in_channels,
                                               int out_channels, int in_h, int in_w, int kernel_h,
                                               int kernel_w, int stride_h, int stride_w, int pad_h,
                                               int pad_w, cudaStream_t stream) {
    CB200_REQUIRE(grad_output != nullptr && weight != nullptr && grad_input != nullptr,
                  "conv2d backward: null tensor pointer");
    const ConvShape s{batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w,
                      stride_h, stride_w, pad_h, pad_w};
    cudeep_b200::check_conv_shape(s);
    // As a forward convolution: input = grad_output [N, OC, OH, OW], filters [C, OC, KH, KW],
    // output = grad_input [N, C, H, W].
    const ConvShape as_forward{batch, out_channels, in_channels, s.out_h(), s.out_w(), kernel_h, kernel_w,
                               1, 1, kernel_h - 1 - pad_h, kernel_w - 1 - pad_w};
    // (As a forward convolution its input channels are this one's output channels; with one or two
    // of them the forward path would need its row-packed form, which flipped filters do not have.)
    const bool pad_fits = pad_h <= kernel_h - 1 && pad_w <= kernel_w - 1 && out_channels >= 3;
    const bool stride_one = stride_h == 1 && stride_w == 1;
    // The fallback form of a strided layer (when the sub-pixel form below does not take it):
    // grad_output with (stride - 1) zeros put between its pixels, and as many zero rows and columns
    // behind it as the forward pass left unread, is the input of the same stride-1 convolution.  The
    // tensor cores then multiply stride_h * stride_w times more zeros than data, which still beats
    // the gather kernel by far up to that factor 16.
    ConvShape dilated = as_forward;
    dilated.in_h = (s.out_h() - 1) * stride_h + 1 + (in_h + 2 * pad_h - kernel_h) % stride_h;
    dilated.in_w = (s.out_w() - 1) * stride_w + 1 + (in_w + 2 * pad_w - kernel_w) % stride_w;
    if (pad_fits && stride_one && cudeep_b200::conv2d_igemm_supported(as_forward)) {
        // The filter packing of the forward path reads the filters flipped and with their
        // channel axes swapped: no re-arranged copy is made.
        cudeep_b200::conv2d_igemm(grad_output, weight, nullptr, grad_input, as_forward, cudeep_b200::EPI_NONE,
                                  stream, /*flipped_filters=*/true);
    } else if (!stride_one && cudeep_b200::conv2d_grad_input_by_parity_supported(s)) {
        // One stride-1 convolution of grad_output per parity class of the input pixels.
        cudeep_b200::conv2d_grad_input_by_parity(grad_output, weight, grad_input, s, stream);
    } else if (pad_fits && !stride_one && stride_h * stride_w <= 16 &&
               cudeep_b200::conv2d_igemm_supported(dilated)) {
        const cudeep_b200::InputDilation dilation{s.out_h(), s.out_w(), stride_h, stride_w};
        cudeep_b200::conv2d_igemm(grad_output, weight, nullptr, grad_input, dilated, cudeep_b200::EPI_NONE,
                                  stream, /*flipped_filters=*/true, &dilation);
    } else {
        cudeep_b200::backward_data_direct<float>(grad_output, weight, grad_input, s, stream);
    }
}

template <>
void launch_conv2d_backward_data_kernel<double>(const double* grad_output, const double* weight,
                                                double* grad_input, int batch, int in_channels,
                                                int out_channels, int in_h, int in_w, int kernel_h,
                                                int kernel_w, int stride_h, int stride_w, int pad_h,
                                                int pad_w, cudaStream_t stream) {
    CB200_REQUIRE(grad_output != nullptr && weight != nullptr && grad_input != nullptr,
                  "conv2d backward: null tensor pointer");
    const ConvShape s{batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w,
                      stride_h, stride_w, pad_h, pad_w};
    cudeep_b200::check_conv_shape(s);
    cudeep_b200::backward_data_direct<double>(grad_output, weight, grad_input, s, stream);
}

template <typename T>
static void backward_weight(const T* grad_output, const T* input, T* grad_weight, const ConvShape& s,
                            cudaStream_t stream) {
    CB200_REQUIRE(grad_output != nullptr && input != nullptr && grad_weight != nullptr,
                  "conv2d backward: null tensor pointer");
    cudeep_b200::check_conv_shape(s);
    const long long total = static_cast<long long>(s.out_c) * s.in_c * s.k_h * s.k_w;
    CB200_TRACE("conv2d grad_weight direct strict %s: N=%d C=%d %dx%d OC=%d, %dx%d stride %dx%d",
                sizeof(T) == 8 ? "FP64" : "FP32", s.batch, s.in_c, s.in_h, s.in_w, s.out_c, s.k_h, s.k_w, s.s_h, s.s_w);
    cudeep_b200::conv2d_backward_weight_direct_kernel<T>
        <<<cudeep_b200::grid_for(total), 256, 0, stream>>>(grad_output, input, grad_weight, s, s.out_h(),
                                                           s.out_w(), total);
    CB200_CHECK_LAUNCH();
}

template <>
void launch_conv2d_backward_weight_kernel<float>(const float* grad_output, const float* input,
                                                 float* grad_weight, int batch, int in_channels,
                                                 int out_channels, int in_h, int in_w, int kernel_h,
                                                 int kernel_w, int stride_h, int stride_w, int pad_h,
                                                 int pad_w, cudaStream_t stream) {
    const ConvShape s{batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w,
                      stride_h, stride_w, pad_h, pad_w};
    CB200_REQUIRE(grad_output != nullptr && input != nullptr && grad_weight != nullptr,
                  "conv2d backward: null tensor pointer");
    cudeep_b200::check_conv_shape(s);
    // Stride-1 shapes with enough channels and pixels: tensor cores (TF32, like the reference's GEMM);
    // everything else: the direct strict-FP32 kernel.
    if (cudeep_b200::conv2d_wgrad_igemm_supported(s))
        cudeep_b200::conv2d_wgrad_igemm(grad_output, input, grad_weight, s, stream);
    else
        backward_weight<float>(grad_output, input, grad_weight, s, stream);
}

template <>
void launch_conv2d_backward_weight_kernel<double>(const double* grad_output, const double* input,
                                                  double* grad_weight, int batch, int in_channels,
                                                  int out_channels, int in_h, int in_w, int kernel_h,
                                                  int kernel_w, int stride_h, int stride_w, int pad_h,
                                                  int pad_w, cudaStream_t stream) {
    backward_weight<double>(grad_output, input, grad_weight,
                            ConvShape{batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w,
                                      stride_h, stride_w, pad_h, pad_w}, stream);
}

}  // namespace kernels
}  // namespace cudeep
