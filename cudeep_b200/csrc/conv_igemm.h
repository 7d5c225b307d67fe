// Host entry of the implicit-GEMM convolution (see conv_igemm.cu).
#pragma once

#include "conv_direct.h"

namespace cudeep_b200 {

// True when the tensor-core path takes this shape: sm_100 device, strides 1..8,
// padding smaller than the filter, at least 32 output channels, at least 3
// input channels (any number when conv2d_igemm_row_packed) and at least 64 output pixels.
bool conv2d_igemm_supported(const ConvShape& s);

// True when a filter row's taps share one 32-wide K block (KW x the channel count rounded up to a
// multiple of 4 is at most 32, KW > 1): only for calls without flipped filters or dilation.
bool conv2d_igemm_row_packed(const ConvShape& s);

// Bytes of scratch one call needs: the NHWC copy of the input followed by the
// packed filters.  The two optional outputs receive the size of each part.
size_t conv2d_igemm_scratch_bytes(const ConvShape& s, size_t* nhwc_bytes, size_t* filter_bytes);

// The input of a launch given in compact form: `input` holds src_h x src_w pixels per channel and
// pixel (r, q) of it stands at (r * d_h, q * d_w) of the in_h x in_w plane the shape describes;
// every other pixel of that plane is zero.  This is how the grad_output of a strided convolution
// enters the stride-1 convolution that yields its grad_input.
struct InputDilation {
    int src_h, src_w, d_h, d_w;
};

// Convolution with caller-provided scratch (256-byte aligned, at least
// conv2d_igemm_scratch_bytes).  force_ctas: 0 = choose, 1 or 2 = CTAs per MMA.
// flipped_filters: `weight` is [C][OC][KH][KW] as seen from `s` (the forward filters of the
// convolution whose grad_input this call computes) and is used with both spatial axes reversed
// and the channel axes swapped.
// input_is_nhwc: `input` is [N][H][W][C] (the layout the kernel gathers from) and is read in place,
// which saves the re-layout pass; needs conv2d_igemm_takes_nhwc_input.  The output is NCHW either way.
void conv2d_igemm_with_scratch(const float* input, const float* weight, const float* bias,
                               float* output, const ConvShape& s, int act, void* scratch,
                               int force_ctas, cudaStream_t stream, bool flipped_filters = false,
                               const InputDilation* dilation = nullptr, bool input_is_nhwc = false);
bool conv2d_igemm_takes_nhwc_input(const float* input, const ConvShape& s);

// Convolution with stream-ordered scratch (cudaMallocAsync / cudaFreeAsync on `stream`).
void conv2d_igemm(const float* input, const float* weight, const float* bias, float* output,
                  const ConvShape& s, int act, cudaStream_t stream, bool flipped_filters = false,
                  const InputDilation* dilation = nullptr, bool input_is_nhwc = false);

// x[N][C][HW] -> xt[N][HW][cx] with cx >= C a multiple of 4 (channels past C are zero).
void nchw_to_nhwc(const float* input, float* xt, int batch, int c, int hw, int cx, cudaStream_t stream);

// x[N][C][H][W] -> xt[N][H][W + 2 * pad_w][cx] with pad_w zero pixels on either side of every row
// (the input layout of the row-packed form).
void nchw_to_nhwc_padded(const float* input, float* xt, int batch, int c, int h, int w, int cx, int pad_w,
                         cudaStream_t stream);

// grad_input of a strided layer (`s` is the forward layer's shape) in its sub-pixel form: the input
// pixels fall into stride_h * stride_w parity classes, each the stride-1 convolution of grad_output
// with the sub-filter of the taps that reach it; all classes are computed as ONE stride-1 convolution
// with (class, channel) pairs as output channels, into dense planes that a second pass weaves into
// grad_input.  No zeros are inserted into grad_output.  Needs at least 32 output channels, padding
// smaller than the filter and the combined convolution on the tensor-core path.
bool conv2d_grad_input_by_parity_supported(const ConvShape& s);
void conv2d_grad_input_by_parity(const float* grad_output, const float* weight, float* grad_input,
                                 const ConvShape& s, cudaStream_t stream);

// grad_weight as an implicit GEMM over output pixels (conv_wgrad.cu): strides 1..8, at least 32
// output channels and 256 output pixels.
bool conv2d_wgrad_igemm_supported(const ConvShape& s);
void conv2d_wgrad_igemm(const float* grad_output, const float* input, float* grad_weight, const ConvShape& s,
                        cudaStream_t stream);

}  // namespace cudeep_b200
