// C++ launchers of the Conv2d forward path, Blackwell (sm_100a) build.
//
// launch_conv2d_forward_kernel keeps the name, argument list and mangled
// symbol of the reference's include/cudeep/kernels/conv.cuh:8-16.  Tensors are
// contiguous: input [N, C, H, W], weight [OC, C, KH, KW], bias [OC] or
// nullptr, output [N, OC, OH, OW] with OH = (H + 2*pad_h - KH) / stride_h + 1.
// The operation is a cross-correlation with zero padding, no dilation, no
// groups.  Launches are asynchronous on `stream`; errors are std::runtime_error.
//
// Which launchers return TF32-rounded results (operands truncated to TF32 by the tensor core,
// FP32 accumulation - what the reference's own GEMM-based paths produce) and which strict FP32:
//   * forward, float: implicit GEMM on tcgen05 (TF32) when strides are 1..8, padding is smaller
//     than the filter, OC >= 32, one image has at least 64 output pixels, and C >= 3 (or fewer
//     channels when a filter row fits one 32-wide K block: KW > 1 and KW * ceil4(C) <= 32).  The
//     input is re-laid as NHWC once per call and gathered tap by tap with TMA, filters are packed
//     [OC][KH*KW][C]; no im2col matrix is materialised.  Every other shape: direct strict FP32.
//   * grad_input, float: at stride 1 the same implicit GEMM applied to grad_output with flipped filters
//     (TF32), under the forward conditions with the roles of C and OC exchanged.  A strided layer with
//     OC >= 32 runs in sub-pixel form: one stride-1 implicit GEMM over grad_output whose output
//     channels are (parity class of the input pixel, channel) pairs, then a pass that weaves the
//     classes into grad_input (TF32; no zeros are inserted).  Strided shapes that form does not take
//     use the stride-1 kernel on a zero-inserted copy (stride_h * stride_w <= 16); otherwise strict FP32.
//   * grad_weight, float: implicit GEMM over output pixels (TF32) for strides 1..8, OC >= 32 and at
//     least 256 output pixels in the batch; otherwise strict FP32.
//   * every double instantiation: direct FP64.
#pragma once

#include <cuda_runtime.h>

#include "../common.cuh"
#include "matmul.cuh"

namespace cudeep {
namespace kernels {

// (reference conv.cuh:8-16, conv_kernel.cu:225-335)
template <typename T>
void launch_conv2d_forward_kernel(const T* input, const T* weight, const T* bias, T* output,
                                  int batch, int in_channels, int out_channels, int in_h, int in_w,
                                  int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h,
                                  int pad_w, cudaStream_t stream = nullptr);

// Gradient w.r.t. the input, grad_input [N, C, H, W] from grad_output [N, OC, OH, OW]
// (reference conv.cuh:18-26; precision per shape as listed at the top of this file).
template <typename T>
void launch_conv2d_backward_data_kernel(const T* grad_output, const T* weight, T* grad_input, int batch,
                                        int in_channels, int out_channels, int in_h, int in_w,
                                        int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h,
                                        int pad_w, cudaStream_t stream = nullptr);

// Gradient w.r.t. the filters, grad_weight [OC, C, KH, KW] (reference conv.cuh:28-36; TF32 on the
// tensor cores for the shapes listed at the top of this file, strict FP32 otherwise).
template <typename T>
void launch_conv2d_backward_weight_kernel(const T* grad_output, const T* input, T* grad_weight, int batch,
                                          int in_channels, int out_channels, int in_h, int in_w,
                                          int kernel_h, int kernel_w, int stride_h, int stride_w,
                                          int pad_h, int pad_w, cudaStream_t stream = nullptr);

// Addition: the same convolution with bias and an activation applied in the
// GEMM epilogue (one pass over the output instead of conv + bias + activation).
void launch_conv2d_forward_fused(const float* input, const float* weight, const float* bias,
                                 float* output, int batch, int in_channels, int out_channels,
                                 int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                 int stride_w, int pad_h, int pad_w, GemmEpilogue epilogue,
                                 cudaStream_t stream = nullptr);

// Addition: the fused convolution for an input already stored channels-last.  `input_layout` is the
// reference's own enum (include/cudeep/common.cuh:10-19): Layout::NCHW is launch_conv2d_forward_fused;
// Layout::NHWC reads input [N, H, W, C] in place - the layout the tensor-core kernel gathers from - and
// so skips the re-layout pass of the NCHW form (about a sixth of that call on a 64 x 256 x 56 x 56
// layer).  Weights stay [OC, C, KH, KW] and the output stays [N, OC, OH, OW].  NHWC needs C % 4 == 0,
// a 16-byte aligned input and a shape the tensor-core path takes (see the top of this file); anything
// else throws instead of falling back.
void launch_conv2d_forward_fused_layout(const float* input, Layout input_layout, const float* weight,
                                        const float* bias, float* output, int batch, int in_channels,
                                        int out_channels, int in_h, int in_w, int kernel_h, int kernel_w,
                                        int stride_h, int stride_w, int pad_h, int pad_w, GemmEpilogue epilogue,
                                        cudaStream_t stream = nullptr);

}  // namespace kernels
}  // namespace cudeep
