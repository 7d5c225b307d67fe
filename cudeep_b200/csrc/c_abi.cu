// extern "C" surface of libcudeep_b200.so (declared in include/cudeep_b200.h).
// Each function forwards to the C++ launcher of the same operation and turns
// exceptions into a status code plus a thread-local message.
#include "cudeep_b200.h"

#include "cudeep/kernels/conv.cuh"
#include "cudeep/kernels/matmul.cuh"
#include "cudeep/memory.cuh"
#include "conv_igemm.h"
#include "gemm_f16.h"
#include "gemm_tf32.h"
#include "abi_error.h"
#include "tensor_ops.h"
#include "cudeep/stream.cuh"
#include "cudeep/dist/sharded_gemm.cuh"

#include <string>
#include <vector>

namespace {

thread_local std::string g_last_error;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return CUDEEP_B200_OK;
    } catch (const std::exception& e) {
        g_last_error = e.what();
    } catch (...) {
        g_last_error = "unknown C++ exception";
    }
    return CUDEEP_B200_ERROR;
}

cudaStream_t as_stream(cudeep_b200_stream_t s) { return static_cast<cudaStream_t>(s); }

cudeep::kernels::GemmEpilogue as_epilogue(int code) {
    CB200_REQUIRE(code >= 0 && code <= 4, "unknown epilogue code");
    return static_cast<cudeep::kernels::GemmEpilogue>(code);
}

// Device buffer from the pool, returned on scope exit.
struct PoolBuffer {
    void* ptr = nullptr;
    explicit PoolBuffer(size_t bytes) : ptr(cudeep::device_malloc(bytes)) {}
    ~PoolBuffer() { cudeep::device_free(ptr); }
    PoolBuffer(const PoolBuffer&) = delete;
    PoolBuffer& operator=(const PoolBuffer&) = delete;
    template <typename T> T* as() const { return static_cast<T*>(ptr); }
};

// One private stream per thread for the host-buffer entry points, so their
// copies and kernels do not serialise against the legacy default stream.
cudaStream_t host_call_stream() {
    thread_local cudaStream_t stream = nullptr;
    thread_local int stream_device = -1;
    int dev = 0;
    CB200_CUDA(cudaGetDevice(&dev));
    if (stream == nullptr || stream_device != dev) {
        CB200_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        stream_device = dev;
    }
    return stream;
}

}  // namespace

namespace cudeep_b200 {
void set_last_error(const std::string& message) { g_last_error = message; }
}  // namespace cudeep_b200

extern "C" {

int cudeep_b200_version(void) { return 100; }

const char* cudeep_b200_last_error(void) { return g_last_error.c_str(); }

int cudeep_b200_device_status(int clear, uint32_t* status) {
    return guarded([&] {
        CB200_REQUIRE(status != nullptr, "status pointer is null");
        *status = cudeep_b200::read_device_status(clear != 0);
    });
}

int cudeep_b200_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K,
                           cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::kernels::launch_matmul_kernel<float>(A, B, C, M, N, K, as_stream(stream)); });
}

int cudeep_b200_matmul_f32_strict(const float* A, const float* B, float* C, int M, int N, int K,
                                  cudeep_b200_stream_t stream) {
    return guarded(
        [&] { cudeep::kernels::launch_matmul_kernel_fp32<float>(A, B, C, M, N, K, as_stream(stream)); });
}

int cudeep_b200_matmul_f64(const double* A, const double* B, double* C, int M, int N, int K,
                           cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::kernels::launch_matmul_kernel<double>(A, B, C, M, N, K, as_stream(stream)); });
}

int cudeep_b200_matmul_fused_act(const float* A, const float* B, float* C, int M, int N, int K,
                                 int epilogue, cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_matmul_fused_act(A, B, C, M, N, K, as_epilogue(epilogue), as_stream(stream));
    });
}

int cudeep_b200_linear_forward_f32(const float* x, const float* W, const float* bias, float* y,
                                   int M, int N, int K, int epilogue, cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_linear_forward(x, W, bias, y, M, N, K, as_epilogue(epilogue), as_stream(stream));
    });
}

int cudeep_b200_linear_forward_f64(const double* x, const double* W, const double* bias, double* y,
                                   int M, int N, int K, int epilogue, cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_linear_forward(x, W, bias, y, M, N, K, as_epilogue(epilogue), as_stream(stream));
    });
}

int cudeep_b200_matmul_nt_f32(const float* A, const float* B, float* C, int M, int N, int K,
                              cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::kernels::launch_matmul_nt(A, B, C, M, N, K, as_stream(stream)); });
}

int cudeep_b200_matmul_tn_f32(const float* A, const float* B, float* C, int M, int N, int K,
                              cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::kernels::launch_matmul_tn(A, B, C, M, N, K, as_stream(stream)); });
}

int cudeep_b200_gemm_tf32_tuned(const float* A, const float* B, int b_is_nk, float* C, int M, int N,
                                int K, const float* bias, int bias_per_row, int epilogue, int ctas,
                                int bn, int raster_group, int max_ctas, uint32_t b_lbo,
                                uint32_t b_sbo, cudeep_b200_stream_t stream) {
    return guarded([&] {
        CB200_REQUIRE(A != nullptr && B != nullptr && C != nullptr, "gemm: null operand pointer");
        CB200_REQUIRE(epilogue >= 0 && epilogue <= 4, "unknown epilogue code");
        cudeep_b200::GemmTuning tune;
        tune.ctas = ctas;
        tune.bn = bn;
        tune.raster_group = raster_group;
        tune.max_ctas = max_ctas & 0xffff;
        tune.stages = (max_ctas >> 16) & 0xff;      // packed: see cudeep_b200.h
        tune.debug = static_cast<uint32_t>(max_ctas >> 24) & 0xfu;
        tune.b_chunked = ((max_ctas >> 28) & 1) ? -1 : 0;
        tune.katoms = (max_ctas >> 29) & 3;
        tune.split_k = static_cast<int>(b_lbo >> 16) & 0xff;      // packed: see cudeep_b200.h
        tune.cluster_split = static_cast<int>(b_lbo >> 24) & 0xf;
        tune.tma_store = ((b_lbo >> 28) & 1u) ? -1 : 0;
        tune.debug |= ((b_lbo >> 29) & 3u) << 4;
        tune.ring_staging = ((b_lbo >> 31) & 1u) ? -1 : 0;
        tune.b_lbo = b_lbo & 0xffffu;
        tune.b_sbo = b_sbo & 0xffffu;
        tune.wait_limit_ms = (b_sbo >> 16) & 0x7fffu;
        if (b_sbo >> 31) tune.debug |= 0x80u;
        cudeep_b200::gemm_tf32(A, B, b_is_nk != 0, C, M, N, K, bias, bias_per_row != 0, epilogue, tune,
                               as_stream(stream));
    });
}

int cudeep_b200_gemm_tf32_plan(int M, int N, int K, int epilogue, int num_sms, int* ctas, int* bn,
                               int* cluster_split, int* katoms, double* estimate_us) {
    return guarded([&] {
        const cudeep_b200::GemmPlan plan = cudeep_b200::gemm_tf32_plan(M, N, K, epilogue, num_sms);
        if (ctas) *ctas = plan.ctas;
        if (bn) *bn = plan.bn;
        if (cluster_split) *cluster_split = plan.cluster_split;
        if (katoms) *katoms = plan.katoms;
        if (estimate_us) *estimate_us = plan.estimate_us;
    });
}

int cudeep_b200_matmul_f16(const void* A, const void* B, float* C, int M, int N, int K,
                           cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_matmul_kernel_fp16(static_cast<const __half*>(A), static_cast<const __half*>(B), C,
                                                   M, N, K, as_stream(stream));
    });
}

int cudeep_b200_matmul_bf16(const void* A, const void* B, float* C, int M, int N, int K,
                            cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_matmul_kernel_bf16(static_cast<const __nv_bfloat16*>(A),
                                                   static_cast<const __nv_bfloat16*>(B), C, M, N, K, as_stream(stream));
    });
}

int cudeep_b200_matmul_f16_tuned(const void* A, const void* B, float* C, int M, int N, int K, int ctas,
                                 uint32_t b_lbo, uint32_t b_sbo, cudeep_b200_stream_t stream) {
    return guarded([&] {
        CB200_REQUIRE(A != nullptr && B != nullptr && C != nullptr, "gemm: null operand pointer");
        cudeep_b200::gemm_f16(static_cast<const __half*>(A), static_cast<const __half*>(B), C, M, N, K, ctas,
                              b_lbo, b_sbo, as_stream(stream));
    });
}

int cudeep_b200_conv2d_forward_f32(const float* input, const float* weight, const float* bias,
                                   float* output, int batch, int in_channels, int out_channels,
                                   int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                   int stride_w, int pad_h, int pad_w, cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_conv2d_forward_kernel<float>(input, weight, bias, output, batch, in_channels,
                                                             out_channels, in_h, in_w, kernel_h, kernel_w,
                                                             stride_h, stride_w, pad_h, pad_w,
                                                             as_stream(stream));
    });
}

int cudeep_b200_conv2d_forward_fused_nhwc_f32(const float* input_nhwc, const float* weight,
                                              const float* bias, float* output, int batch,
                                              int in_channels, int out_channels, int in_h, int in_w,
                                              int kernel_h, int kernel_w, int stride_h, int stride_w,
                                              int pad_h, int pad_w, int epilogue,
                                              cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_conv2d_forward_fused_layout(
            input_nhwc, cudeep::Layout::NHWC, weight, bias, output, batch, in_channels, out_channels, in_h, in_w,
            kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, as_epilogue(epilogue), as_stream(stream));
    });
}

int cudeep_b200_conv2d_forward_fused_f32(const float* input, const float* weight, const float* bias,
                                         float* output, int batch, int in_channels, int out_channels,
                                         int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                         int stride_w, int pad_h, int pad_w, int epilogue,
                                         cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_conv2d_forward_fused(input, weight, bias, output, batch, in_channels,
                                                     out_channels, in_h, in_w, kernel_h, kernel_w, stride_h,
                                                     stride_w, pad_h, pad_w, as_epilogue(epilogue),
                                                     as_stream(stream));
    });
}

int cudeep_b200_conv2d_forward_f64(const double* input, const double* weight, const double* bias,
                                   double* output, int batch, int in_channels, int out_channels,
                                   int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                   int stride_w, int pad_h, int pad_w, cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_conv2d_forward_kernel<double>(input, weight, bias, output, batch, in_channels,
                                                              out_channels, in_h, in_w, kernel_h, kernel_w,
                                                              stride_h, stride_w, pad_h, pad_w,
                                                              as_stream(stream));
    });
}

int cudeep_b200_conv2d_backward_data_f32(const float* grad_output, const float* weight, float* grad_input,
                                         int batch, int in_channels, int out_channels, int in_h, int in_w,
                                         int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h,
                                         int pad_w, cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_conv2d_backward_data_kernel<float>(
            grad_output, weight, grad_input, batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w,
            stride_h, stride_w, pad_h, pad_w, as_stream(stream));
    });
}

int cudeep_b200_conv2d_backward_weight_f32(const float* grad_output, const float* input, float* grad_weight,
                                           int batch, int in_channels, int out_channels, int in_h, int in_w,
                                           int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h,
                                           int pad_w, cudeep_b200_stream_t stream) {
    return guarded([&] {
        cudeep::kernels::launch_conv2d_backward_weight_kernel<float>(
            grad_output, input, grad_weight, batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w,
            stride_h, stride_w, pad_h, pad_w, as_stream(stream));
    });
}

// ---------------------------------------------------------------- host-buffer entry points

}  // extern "C"

namespace {

// Streams and events of the pipelined host matmul, one set per thread and device.
struct HostPipeline {
    cudaStream_t in = nullptr, compute = nullptr, out = nullptr;
    std::vector<cudaEvent_t> events;
    int device = -1;
    cudaEvent_t event(size_t i) {
        while (events.size() <= i) {
            cudaEvent_t e = nullptr;
            CB200_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            events.push_back(e);
        }
        return events[i];
    }
};

HostPipeline& host_pipeline() {
    thread_local HostPipeline p;
    int dev = 0;
    CB200_CUDA(cudaGetDevice(&dev));
    if (p.device != dev) {
        p = HostPipeline{};
        CB200_CUDA(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
        CB200_CUDA(cudaStreamCreateWithFlags(&p.compute, cudaStreamNonBlocking));
        CB200_CUDA(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
        p.device = dev;
    }
    return p;
}

}  // namespace

extern "C" {

int cudeep_b200_matmul_host_f32(const float* A, const float* B, float* C, int M, int N, int K, int strict) {
    return guarded([&] {
        CB200_REQUIRE(A != nullptr && B != nullptr && C != nullptr, "matmul: null host pointer");
        CB200_REQUIRE(M > 0 && N > 0 && K > 0, "matmul: M, N and K must be positive");
        const size_t a_bytes = size_t(M) * K * sizeof(float);
        const size_t b_bytes = size_t(K) * N * sizeof(float);
        const size_t c_bytes = size_t(M) * N * sizeof(float);
        PoolBuffer da(a_bytes), db(b_bytes), dc(c_bytes);
        // The host link, not the GEMM, bounds this call.  B goes up first (every row of C needs
        // all of it); A then goes up in row bands, each band is multiplied as soon as it has
        // landed, and its rows of C go back down while later bands are still going up, so the
        // two directions of the link and the tensor cores all work at once.
        int bands = 1;
        const size_t band_target = size_t(32) << 20;
        if (a_bytes + c_bytes > 4 * band_target) {
            bands = static_cast<int>((a_bytes + c_bytes) / 2 / band_target);
            if (bands > 32) bands = 32;
            if (bands < 1) bands = 1;
        }
        int band_rows = (M + bands - 1) / bands;
        band_rows = (band_rows + 255) / 256 * 256;          // whole 256-row tiles per band
        HostPipeline& p = host_pipeline();
        cudeep::memcpy_h2d(db.ptr, B, b_bytes, p.in);
        size_t ev = 0;
        for (int row0 = 0; row0 < M; row0 += band_rows) {
            const int rows = (M - row0 < band_rows) ? (M - row0) : band_rows;
            float* a_dev = da.as<float>() + size_t(row0) * K;
            float* c_dev = dc.as<float>() + size_t(row0) * N;
            cudeep::memcpy_h2d(a_dev, A + size_t(row0) * K, size_t(rows) * K * sizeof(float), p.in);
            cudaEvent_t landed = p.event(ev++);
            CB200_CUDA(cudaEventRecord(landed, p.in));
            CB200_CUDA(cudaStreamWaitEvent(p.compute, landed, 0));
            if (strict)
                cudeep::kernels::launch_matmul_kernel_fp32<float>(a_dev, db.as<float>(), c_dev, rows, N, K,
                                                                  p.compute);
            else
                cudeep::kernels::launch_matmul_kernel<float>(a_dev, db.as<float>(), c_dev, rows, N, K, p.compute);
            cudaEvent_t done = p.event(ev++);
            CB200_CUDA(cudaEventRecord(done, p.compute));
            CB200_CUDA(cudaStreamWaitEvent(p.out, done, 0));
            cudeep::memcpy_d2h(C + size_t(row0) * N, c_dev, size_t(rows) * N * sizeof(float), p.out);
        }
        CB200_CUDA(cudaStreamSynchronize(p.out));
        CB200_CUDA(cudaStreamSynchronize(p.compute));
        CB200_CUDA(cudaStreamSynchronize(p.in));
    });
}

int cudeep_b200_linear_forward_host_f32(const float* x, const float* W, const float* bias, float* y,
                                        int M, int N, int K, int epilogue) {
    return guarded([&] {
        CB200_REQUIRE(x != nullptr && W != nullptr && y != nullptr, "linear: null host pointer");
        CB200_REQUIRE(M > 0 && N > 0 && K > 0, "linear: M, N and K must be positive");
        const size_t x_bytes = size_t(M) * K * sizeof(float);
        const size_t w_bytes = size_t(N) * K * sizeof(float);
        const size_t y_bytes = size_t(M) * N * sizeof(float);
        PoolBuffer dx(x_bytes), dw(w_bytes), dy(y_bytes), dbias(size_t(N) * sizeof(float));
        cudaStream_t s = host_call_stream();
        cudeep::memcpy_h2d(dx.ptr, x, x_bytes, s);
        cudeep::memcpy_h2d(dw.ptr, W, w_bytes, s);
        if (bias != nullptr) cudeep::memcpy_h2d(dbias.ptr, bias, size_t(N) * sizeof(float), s);
        cudeep::kernels::launch_linear_forward(dx.as<float>(), dw.as<float>(),
                                               bias != nullptr ? dbias.as<float>() : nullptr,
                                               dy.as<float>(), M, N, K, as_epilogue(epilogue), s);
        cudeep::memcpy_d2h(y, dy.ptr, y_bytes, s);
        CB200_CUDA(cudaStreamSynchronize(s));
    });
}

int cudeep_b200_conv2d_forward_host_f32(const float* input, const float* weight, const float* bias,
                                        float* output, int batch, int in_channels, int out_channels,
                                        int in_h, int in_w, int kernel_h, int kernel_w, int stride_h,
                                        int stride_w, int pad_h, int pad_w, int epilogue) {
    return guarded([&] {
        CB200_REQUIRE(input != nullptr && weight != nullptr && output != nullptr,
                      "conv2d: null host pointer");
        const cudeep_b200::ConvShape shape{batch, in_channels, out_channels, in_h, in_w, kernel_h,
                                           kernel_w, stride_h, stride_w, pad_h, pad_w};
        cudeep_b200::check_conv_shape(shape);
        const size_t x_bytes = size_t(batch) * in_channels * in_h * in_w * sizeof(float);
        const size_t w_bytes = size_t(out_channels) * in_channels * kernel_h * kernel_w * sizeof(float);
        const size_t y_bytes = size_t(batch) * out_channels * shape.out_h() * shape.out_w() * sizeof(float);
        PoolBuffer dx(x_bytes), dw(w_bytes), dy(y_bytes), dbias(size_t(out_channels) * sizeof(float));
        cudaStream_t s = host_call_stream();
        cudeep::memcpy_h2d(dx.ptr, input, x_bytes, s);
        cudeep::memcpy_h2d(dw.ptr, weight, w_bytes, s);
        if (bias != nullptr) cudeep::memcpy_h2d(dbias.ptr, bias, size_t(out_channels) * sizeof(float), s);
        cudeep::kernels::launch_conv2d_forward_fused(dx.as<float>(), dw.as<float>(),
                                                     bias != nullptr ? dbias.as<float>() : nullptr,
                                                     dy.as<float>(), batch, in_channels, out_channels, in_h,
                                                     in_w, kernel_h, kernel_w, stride_h, stride_w, pad_h,
                                                     pad_w, as_epilogue(epilogue), s);
        cudeep::memcpy_d2h(output, dy.ptr, y_bytes, s);
        CB200_CUDA(cudaStreamSynchronize(s));
    });
}

// ---------------------------------------------------------------- tensor plumbing

int cudeep_b200_memcpy_h2d(void* dst, const void* src, size_t nbytes, cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::memcpy_h2d(dst, src, nbytes, as_stream(stream)); });
}
int cudeep_b200_memcpy_d2h(void* dst, const void* src, size_t nbytes, cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::memcpy_d2h(dst, src, nbytes, as_stream(stream)); });
}
int cudeep_b200_memcpy_d2d(void* dst, const void* src, size_t nbytes, cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::memcpy_d2d(dst, src, nbytes, as_stream(stream)); });
}
int cudeep_b200_stream_synchronize(cudeep_b200_stream_t stream) {
    return guarded([&] { CB200_CUDA(cudaStreamSynchronize(as_stream(stream))); });
}
int cudeep_b200_device_synchronize(void) {
    return guarded([&] { CB200_CUDA(cudaDeviceSynchronize()); });
}

int cudeep_b200_strided_copy(const void* src, void* dst, int ndim, const long long* shape,
                             const long long* strides, int elem_size, cudeep_b200_stream_t stream) {
    return guarded([&] {
        CB200_REQUIRE(src != nullptr && dst != nullptr && shape != nullptr && strides != nullptr,
                      "strided copy: null pointer");
        CB200_REQUIRE(ndim >= 1 && ndim <= cudeep_b200::StridedView::kMaxDims, "strided copy: rank must be 1..8");
        cudeep_b200::StridedView view{};
        view.ndim = ndim;
        for (int d = 0; d < ndim; ++d) {
            view.shape[d] = shape[d];
            view.strides[d] = strides[d];
        }
        if (elem_size == 4)
            cudeep_b200::strided_copy<float>(static_cast<const float*>(src), static_cast<float*>(dst), view,
                                             as_stream(stream));
        else if (elem_size == 8)
            cudeep_b200::strided_copy<double>(static_cast<const double*>(src), static_cast<double*>(dst), view,
                                              as_stream(stream));
        else
            CB200_REQUIRE(false, "strided copy: element size must be 4 or 8");
    });
}

int cudeep_b200_fill_f32(float* dst, float value, long long count, cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep_b200::fill<float>(dst, value, count, as_stream(stream)); });
}
int cudeep_b200_fill_f64(double* dst, double value, long long count, cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep_b200::fill<double>(dst, value, count, as_stream(stream)); });
}

int cudeep_b200_broadcast_add_f32(const float* matrix, const float* row, float* out, long long rows, int cols,
                                  cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep_b200::add_row<float>(matrix, row, out, rows, cols, as_stream(stream)); });
}
int cudeep_b200_broadcast_add_f64(const double* matrix, const double* row, double* out, long long rows,
                                  int cols, cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep_b200::add_row<double>(matrix, row, out, rows, cols, as_stream(stream)); });
}

int cudeep_b200_activation_f32(const float* x, float* y, long long count, int epilogue,
                               cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep_b200::activation(x, y, count, epilogue, as_stream(stream)); });
}

// ---------------------------------------------------------------- streams and events

int cudeep_b200_stream_create(cudeep_b200_stream_t* stream) {
    return guarded([&] {
        CB200_REQUIRE(stream != nullptr, "stream_create: null result pointer");
        cudeep::Stream s;
        *stream = s.release();
    });
}
int cudeep_b200_stream_destroy(cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::Stream::destroy_handle(as_stream(stream)); });
}
int cudeep_b200_event_create(void** event) {
    return guarded([&] {
        CB200_REQUIRE(event != nullptr, "event_create: null result pointer");
        cudaEvent_t e = nullptr;
        CB200_CUDA(cudaEventCreate(&e));
        *event = e;
    });
}
int cudeep_b200_event_destroy(void* event) {
    return guarded([&] { CB200_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event))); });
}
int cudeep_b200_event_record(void* event, cudeep_b200_stream_t stream) {
    return guarded([&] { CB200_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), as_stream(stream))); });
}
int cudeep_b200_event_synchronize(void* event) {
    return guarded([&] { CB200_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event))); });
}
int cudeep_b200_event_elapsed_ms(void* start, void* end, float* ms) {
    return guarded([&] {
        CB200_REQUIRE(ms != nullptr, "event_elapsed_ms: null result pointer");
        CB200_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(end)));
    });
}

int cudeep_b200_device_info(int* device, int* sm_count, int* cc_major, int* cc_minor, size_t* total_mem) {
    return guarded([&] {
        const cudeep_b200::DeviceInfo& info = cudeep_b200::device_info();
        if (device) *device = info.device;
        if (sm_count) *sm_count = info.num_sms;
        if (cc_major) *cc_major = info.cc_major;
        if (cc_minor) *cc_minor = info.cc_minor;
        if (total_mem) {
            size_t free_b = 0, total_b = 0;
            CB200_CUDA(cudaMemGetInfo(&free_b, &total_b));
            *total_mem = total_b;
        }
    });
}

// ---------------------------------------------------------------- memory pool

int cudeep_b200_pool_alloc(size_t nbytes, void** ptr) {
    return guarded([&] {
        CB200_REQUIRE(ptr != nullptr, "pool_alloc: null result pointer");
        *ptr = cudeep::device_malloc(nbytes);
    });
}

int cudeep_b200_pool_free(void* ptr) {
    return guarded([&] { cudeep::device_free(ptr); });
}

int cudeep_b200_pool_alloc_on_stream(size_t nbytes, cudeep_b200_stream_t stream, void** ptr) {
    return guarded([&] {
        CB200_REQUIRE(ptr != nullptr, "pool_alloc: null result pointer");
        *ptr = cudeep::MemoryPool::instance().allocate(nbytes, as_stream(stream));
    });
}

int cudeep_b200_pool_free_on_stream(void* ptr, cudeep_b200_stream_t stream) {
    return guarded([&] { cudeep::device_free(ptr, as_stream(stream)); });
}

int cudeep_b200_pool_release_cached(void) {
    return guarded([&] { cudeep::MemoryPool::instance().release_cached(); });
}

int cudeep_b200_pool_stats(size_t* allocated_bytes, size_t* cached_bytes) {
    return guarded([&] {
        cudeep::MemoryPool& pool = cudeep::MemoryPool::instance();
        if (allocated_bytes) *allocated_bytes = pool.allocated_bytes();
        if (cached_bytes) *cached_bytes = pool.cached_bytes();
    });
}

int cudeep_b200_scratch_trim(size_t keep_bytes) {
    return guarded([&] { cudeep_b200::scratch_trim(keep_bytes); });
}

// ---------------------------------------------------------------- row-sharded GEMM

namespace {
cudeep::dist::ShardedGemm& sharded(cudeep_b200_sharded_gemm_t g) {
    CB200_REQUIRE(g != nullptr, "sharded GEMM handle is null");
    return *reinterpret_cast<cudeep::dist::ShardedGemm*>(g);
}
cudeep::dist::ShardedGemmOptions sharded_options(int bands, int comm_sms, int dry_run) {
    cudeep::dist::ShardedGemmOptions opt;
    if (bands > 0) opt.bands = bands;
    if (comm_sms >= 0) opt.comm_sms = comm_sms;
    opt.dry_run = (dry_run & 1) != 0;        // `dry_run` is a flag word: bit 0 dry run, bit 1 multicast
    opt.multicast = (dry_run & 2) != 0;
    return opt;
}
}  // namespace

int cudeep_b200_sharded_gemm_create_local(const int* devices, int n_devices, long long M, int N, int K,
                                          int bands, int comm_sms, int dry_run,
                                          cudeep_b200_sharded_gemm_t* out) {
    return guarded([&] {
        CB200_REQUIRE(devices != nullptr && n_devices > 0 && out != nullptr, "sharded_gemm_create_local: bad arguments");
        const std::vector<int> list(devices, devices + n_devices);
        *out = reinterpret_cast<cudeep_b200_sharded_gemm_t>(
            new cudeep::dist::ShardedGemm(list, M, N, K, sharded_options(bands, comm_sms, dry_run)));
    });
}

int cudeep_b200_sharded_gemm_create_rank(int rank, int world, int device, long long M, int N, int K,
                                         int bands, int comm_sms, int dry_run,
                                         cudeep_b200_sharded_gemm_t* out) {
    return guarded([&] {
        CB200_REQUIRE(out != nullptr, "sharded_gemm_create_rank: null result pointer");
        *out = reinterpret_cast<cudeep_b200_sharded_gemm_t>(
            new cudeep::dist::ShardedGemm(rank, world, device, M, N, K, sharded_options(bands, comm_sms, dry_run)));
    });
}

int cudeep_b200_sharded_gemm_destroy(cudeep_b200_sharded_gemm_t g) {
    return guarded([&] { delete reinterpret_cast<cudeep::dist::ShardedGemm*>(g); });
}

int cudeep_b200_sharded_gemm_rows(cudeep_b200_sharded_gemm_t g, int rank, int band, long long* row0,
                                  long long* rows) {
    return guarded([&] {
        const cudeep::dist::RowRange r = band < 0 ? sharded(g).rows_of(rank) : sharded(g).band_of(rank, band);
        if (row0) *row0 = r.row0;
        if (rows) *rows = r.rows;
    });
}

int cudeep_b200_sharded_gemm_buffers(cudeep_b200_sharded_gemm_t g, int local, float** a_shard, float** b,
                                     float** c) {
    return guarded([&] {
        if (a_shard) *a_shard = sharded(g).a_shard(local);
        if (b) *b = sharded(g).b(local);
        if (c) *c = sharded(g).c(local);
    });
}

int cudeep_b200_sharded_gemm_read_c(cudeep_b200_sharded_gemm_t g, int local, long long row0, long long rows,
                                    float* host_dst) {
    return guarded([&] { sharded(g).read_c(local, row0, rows, host_dst); });
}

int cudeep_b200_sharded_gemm_comm_id(void* id_out) {
    return guarded([&] { cudeep::dist::ShardedGemm::new_comm_id(id_out); });
}

int cudeep_b200_sharded_gemm_init_comm(cudeep_b200_sharded_gemm_t g, const void* id) {
    return guarded([&] { sharded(g).init_comm(id); });
}

int cudeep_b200_sharded_gemm_export_c(cudeep_b200_sharded_gemm_t g, void* handle_out) {
    return guarded([&] { sharded(g).export_c(handle_out); });
}

int cudeep_b200_sharded_gemm_open_peers(cudeep_b200_sharded_gemm_t g, const void* handles) {
    return guarded([&] { sharded(g).open_peers(handles); });
}

int cudeep_b200_sharded_gemm_multicast_fd(cudeep_b200_sharded_gemm_t g, int* fd) {
    return guarded([&] {
        CB200_REQUIRE(fd != nullptr, "sharded_gemm_multicast_fd: null result pointer");
        *fd = sharded(g).multicast_create_fd();
    });
}

int cudeep_b200_sharded_gemm_multicast_join(cudeep_b200_sharded_gemm_t g, int fd) {
    return guarded([&] { sharded(g).multicast_join(fd); });
}

int cudeep_b200_sharded_gemm_multicast_bind(cudeep_b200_sharded_gemm_t g) {
    return guarded([&] { sharded(g).multicast_bind(); });
}

int cudeep_b200_sharded_gemm_run(cudeep_b200_sharded_gemm_t g, int gather, cudeep_b200_stream_t stream) {
    return guarded([&] { sharded(g).run(static_cast<cudeep::dist::Gather>(gather), as_stream(stream)); });
}

int cudeep_b200_sharded_gemm_synchronize(cudeep_b200_sharded_gemm_t g) {
    return guarded([&] { sharded(g).synchronize(); });
}

int cudeep_b200_sharded_gemm_time(cudeep_b200_sharded_gemm_t g, int gather, int steps, int warmup,
                                  float* ms_per_step) {
    return guarded([&] {
        CB200_REQUIRE(ms_per_step != nullptr, "sharded_gemm_time: null result pointer");
        *ms_per_step = sharded(g).time_steps(static_cast<cudeep::dist::Gather>(gather), steps, warmup);
    });
}

int cudeep_b200_sharded_gemm_steps(cudeep_b200_sharded_gemm_t g, int local, long long* steps) {
    return guarded([&] {
        CB200_REQUIRE(steps != nullptr, "sharded_gemm_steps: null result pointer");
        *steps = sharded(g).steps_enqueued(local);
    });
}

int cudeep_b200_sharded_gemm_inject_failure(cudeep_b200_sharded_gemm_t g, int rank) {
    return guarded([&] { sharded(g).inject_failure(rank); });
}

}  // extern "C"
