// Direct convolution: NCHW input, OIHW filters, cross-correlation, zero padding.
// Semantics follow the reference's conv2d_forward_naive_kernel
// (src/kernels/conv_kernel.cu:113-159).  Used for FP64, for strided
// convolutions and for shapes the tensor-core path does not take.  The sum
// runs over (c, kh, kw) in ascending order with fused multiply-adds.
#include "conv_direct.h"
#include "epilogue_math.cuh"

namespace cudeep_b200 {

void check_conv_shape(const ConvShape& s) {
    CB200_REQUIRE(s.batch > 0 && s.in_c > 0 && s.out_c > 0 && s.in_h > 0 && s.in_w > 0,
                  "conv2d: batch, channels and image size must be positive");
    CB200_REQUIRE(s.k_h > 0 && s.k_w > 0 && s.s_h > 0 && s.s_w > 0 && s.p_h >= 0 && s.p_w >= 0,
                  "conv2d: kernel and stride must be positive, padding non-negative");
    CB200_REQUIRE(s.in_h + 2 * s.p_h >= s.k_h && s.in_w + 2 * s.p_w >= s.k_w,
                  "conv2d: kernel larger than the padded input");
}

namespace {

template <typename T> __device__ __forceinline__ T conv_fma(T a, T b, T c);
template <> __device__ __forceinline__ float conv_fma<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double conv_fma<double>(double a, double b, double c) { return fma(a, b, c); }

template <typename T> __device__ __forceinline__ T conv_act(T x, int act);
template <> __device__ __forceinline__ float conv_act<float>(float x, int act) { return apply_activation1(x, act); }
template <> __device__ __forceinline__ double conv_act<double>(double x, int act) {
    switch (act) {
        case EPI_RELU: return x > 0.0 ? x : 0.0;
        case EPI_GELU: return 0.5 * x * (1.0 + tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)));
        case EPI_SILU: return x / (1.0 + exp(-x));
        case EPI_SIGMOID: return 1.0 / (1.0 + exp(-x));
        default: return x;
    }
}

template <typename T>
__global__ void conv2d_direct_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                     const T* __restrict__ bias, T* __restrict__ y, ConvShape s,
                                     int oh_n, int ow_n, long long total, int act) {
    for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int ow = static_cast<int>(idx % ow_n);
        long long r = idx / ow_n;
        const int oh = static_cast<int>(r % oh_n);
        r /= oh_n;
        const int oc = static_cast<int>(r % s.out_c);
        const int n = static_cast<int>(r / s.out_c);
        T acc = T(0);
        for (int c = 0; c < s.in_c; ++c) {
            const T* xc = x + (static_cast<long long>(n) * s.in_c + c) * s.in_h * s.in_w;
            const T* wc = w + (static_cast<long long>(oc) * s.in_c + c) * s.k_h * s.k_w;
            for (int kh = 0; kh < s.k_h; ++kh) {
                const int ih = oh * s.s_h - s.p_h + kh;
                if (ih < 0 || ih >= s.in_h) continue;
                for (int kw = 0; kw < s.k_w; ++kw) {
                    const int iw = ow * s.s_w - s.p_w + kw;
                    if (iw < 0 || iw >= s.in_w) continue;
                    acc = conv_fma<T>(xc[ih * s.in_w + iw], wc[kh * s.k_w + kw], acc);
                }
            }
        }
        if (bias != nullptr) acc += bias[oc];
        y[idx] = conv_act<T>(acc, act);
    }
}

}  // namespace

template <typename T>
void conv2d_direct(const T* input, const T* weight, const T* bias, T* output, const ConvShape& s,
                   int act, cudaStream_t stream) {
    check_conv_shape(s);
    const int oh = s.out_h(), ow = s.out_w();
    const long long total = static_cast<long long>(s.batch) * s.out_c * oh * ow;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    const long long cap = static_cast<long long>(device_info().num_sms) * 32;
    if (blocks > cap) blocks = cap;
    CB200_TRACE("conv2d direct strict %s: N=%d C=%d %dx%d -> OC=%d %dx%d, %dx%d stride %dx%d pad %dx%d, blocks=%lld",
                sizeof(T) == 8 ? "FP64" : "FP32", s.batch, s.in_c, s.in_h, s.in_w, s.out_c, oh, ow, s.k_h, s.k_w, s.s_h,
                s.s_w, s.p_h, s.p_w, blocks);
    conv2d_direct_kernel<T><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        input, weight, bias, output, s, oh, ow, total, act);
    CB200_CHECK_LAUNCH();
}

template void conv2d_direct<float>(const float*, const float*, const float*, float*,
                                   const ConvShape&, int, cudaStream_t);
template void conv2d_direct<double>(const double*, const double*, const double*, double*,
                                    const ConvShape&, int, cudaStream_t);

}  // namespace cudeep_b200
