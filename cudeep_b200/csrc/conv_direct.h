// Direct (one thread per output element) convolution in strict element precision.
#pragma once

#include "runtime.h"

namespace cudeep_b200 {

struct ConvShape {
    int batch, in_c, out_c, in_h, in_w, k_h, k_w, s_h, s_w, p_h, p_w;
    int out_h() const { return (in_h + 2 * p_h - k_h) / s_h + 1; }
    int out_w() const { return (in_w + 2 * p_w - k_w) / s_w + 1; }
};

void check_conv_shape(const ConvShape& s);

template <typename T>
void conv2d_direct(const T* input, const T* weight, const T* bias, T* output, const ConvShape& s,
                   int act, cudaStream_t stream);

}  // namespace cudeep_b200
