// cudeep::Tensor (see include/cudeep/tensor.cuh).
#include "cudeep/tensor.cuh"

#include "cudeep/kernels/matmul.cuh"
#include "cudeep/memory.cuh"
#include "runtime.h"
#include "tensor_ops.h"

#include <atomic>
#include <random>

namespace cudeep {

// Device storage shared by a tensor and its views.  It remembers the stream its owner works
// on, so that the pool hands the block to other streams only after that work has drained.
struct Tensor::Buffer {
    void* ptr = nullptr;
    cudaStream_t stream = nullptr;
    Buffer(size_t bytes, cudaStream_t s) : ptr(device_malloc(bytes > 0 ? bytes : 1, s)), stream(s) {}
    ~Buffer() {
        try {
            device_free(ptr, stream);
        } catch (...) {      // a destructor must not throw; the pool's release path does not, this is belt and braces
        }
    }
    Buffer(const Buffer&) = delete;
    Buffer& operator=(const Buffer&) = delete;
};

namespace {

__global__ void binary_kernel_f32(const float* a, const float* b, float* out, long long n, int op) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = op == 0 ? a[i] + b[i] : op == 1 ? a[i] - b[i] : a[i] * b[i];
}
__global__ void binary_kernel_f64(const double* a, const double* b, double* out, long long n, int op) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = op == 0 ? a[i] + b[i] : op == 1 ? a[i] - b[i] : a[i] * b[i];
}

std::atomic<uint64_t> g_randn_counter{0x9e3779b97f4a7c15ull};

}  // namespace

Tensor::Tensor() = default;

Tensor::Tensor(const std::vector<int64_t>& shape, DType dtype) : Tensor(shape, dtype, nullptr) {}

Tensor::Tensor(const std::vector<int64_t>& shape, DType dtype, cudaStream_t stream)
    : shape_(shape), dtype_(dtype), stream_(stream) {
    for (int64_t s : shape_) CB200_REQUIRE(s >= 0, "Tensor: negative extent");
    compute_strides();
    buffer_ = std::make_shared<Buffer>(nbytes(), stream);
}

void Tensor::set_stream(cudaStream_t stream) {
    stream_ = stream;
    if (buffer_) buffer_->stream = stream;
}

Tensor::Tensor(const Tensor& other)
    : shape_(other.shape_), dtype_(other.dtype_), stream_(other.stream_) {
    compute_strides();
    if (other.buffer_) {
        buffer_ = std::make_shared<Buffer>(nbytes(), stream_);
        const Tensor src = other.is_contiguous() ? Tensor() : other.contiguous();
        const void* from = other.is_contiguous() ? other.data() : src.data();
        memcpy_d2d(buffer_->ptr, from, nbytes(), stream_);
    }
}

Tensor& Tensor::operator=(const Tensor& other) {
    if (this != &other) {
        Tensor copy(other);
        *this = std::move(copy);
    }
    return *this;
}

void* Tensor::data() const { return buffer_ ? buffer_->ptr : nullptr; }

int64_t Tensor::numel() const {
    int64_t n = 1;
    for (int64_t s : shape_) n *= s;
    return n;
}

size_t Tensor::nbytes() const { return static_cast<size_t>(numel()) * dtype_size(dtype_); }

void Tensor::compute_strides() {
    strides_.assign(shape_.size(), 1);
    for (int i = static_cast<int>(shape_.size()) - 2; i >= 0; --i) strides_[i] = strides_[i + 1] * shape_[i + 1];
}

bool Tensor::is_contiguous() const {
    int64_t expect = 1;
    for (int i = static_cast<int>(shape_.size()) - 1; i >= 0; --i) {
        if (shape_[i] != 1 && strides_[i] != expect) return false;
        expect *= shape_[i];
    }
    return true;
}

Tensor Tensor::zeros(const std::vector<int64_t>& shape, DType dtype) {
    Tensor t(shape, dtype);
    t.zero_();
    return t;
}

Tensor Tensor::ones(const std::vector<int64_t>& shape, DType dtype) {
    Tensor t(shape, dtype);
    t.fill_(1.0f);
    return t;
}

Tensor Tensor::randn(const std::vector<int64_t>& shape, DType dtype) {
    return randn_seeded(shape, dtype, g_randn_counter.fetch_add(0x632be59bd9b4e019ull));
}

Tensor Tensor::randn_seeded(const std::vector<int64_t>& shape, DType dtype, uint64_t seed) {
    CB200_REQUIRE(dtype == DType::Float32 || dtype == DType::Float64, "randn: float32 or float64 only");
    Tensor t(shape, dtype);
    const int64_t n = t.numel();
    std::mt19937_64 gen(seed);
    if (dtype == DType::Float32) {
        std::normal_distribution<float> dist(0.0f, 1.0f);
        std::vector<float> host(static_cast<size_t>(n));
        for (auto& v : host) v = dist(gen);
        memcpy_h2d(t.data(), host.data(), t.nbytes(), nullptr);
    } else {
        std::normal_distribution<double> dist(0.0, 1.0);
        std::vector<double> host(static_cast<size_t>(n));
        for (auto& v : host) v = dist(gen);
        memcpy_h2d(t.data(), host.data(), t.nbytes(), nullptr);
    }
    return t;
}

Tensor Tensor::from_host(const void* host_data, const std::vector<int64_t>& shape, DType dtype) {
    CB200_REQUIRE(host_data != nullptr, "from_host: null pointer");
    Tensor t(shape, dtype);
    memcpy_h2d(t.data(), host_data, t.nbytes(), nullptr);   // blocking, as in the reference (tensor.cu:208-212)
    return t;
}

void Tensor::to_host(void* host_dst) const {
    CB200_REQUIRE(host_dst != nullptr, "to_host: null pointer");
    if (numel() == 0) return;
    if (stream_ != nullptr) CB200_CUDA(cudaStreamSynchronize(stream_));
    if (is_contiguous()) {
        memcpy_d2h(host_dst, data(), nbytes(), nullptr);
    } else {
        const Tensor c = contiguous();
        if (stream_ != nullptr) CB200_CUDA(cudaStreamSynchronize(stream_));
        memcpy_d2h(host_dst, c.data(), nbytes(), nullptr);
    }
}

Tensor Tensor::reshape(const std::vector<int64_t>& new_shape) const {
    std::vector<int64_t> shape = new_shape;
    int64_t known = 1;
    int infer = -1;
    for (size_t i = 0; i < shape.size(); ++i) {
        if (shape[i] == -1) {
            CB200_REQUIRE(infer < 0, "reshape: more than one -1");
            infer = static_cast<int>(i);
        } else {
            known *= shape[i];
        }
    }
    if (infer >= 0) shape[infer] = known > 0 ? numel() / known : 0;
    int64_t n = 1;
    for (int64_t s : shape) n *= s;
    CB200_REQUIRE(n == numel(), "reshape: element count mismatch");
    const Tensor base = is_contiguous() ? Tensor() : contiguous();
    Tensor out;
    out.buffer_ = is_contiguous() ? buffer_ : base.buffer_;
    out.shape_ = shape;
    out.dtype_ = dtype_;
    out.stream_ = stream_;
    out.compute_strides();
    return out;
}

Tensor Tensor::transpose(int dim0, int dim1) const {
    const int nd = static_cast<int>(ndim());
    CB200_REQUIRE(dim0 >= -nd && dim0 < nd && dim1 >= -nd && dim1 < nd, "transpose: dimension out of range");
    if (dim0 < 0) dim0 += nd;
    if (dim1 < 0) dim1 += nd;
    Tensor out;
    out.buffer_ = buffer_;
    out.shape_ = shape_;
    out.strides_ = strides_;
    out.dtype_ = dtype_;
    out.stream_ = stream_;
    std::swap(out.shape_[dim0], out.shape_[dim1]);
    std::swap(out.strides_[dim0], out.strides_[dim1]);
    return out;
}

Tensor Tensor::contiguous() const {
    if (is_contiguous()) {
        Tensor out;                       // same buffer, no copy (the reference deep-copies here)
        out.buffer_ = buffer_;
        out.shape_ = shape_;
        out.strides_ = strides_;
        out.dtype_ = dtype_;
        out.stream_ = stream_;
        return out;
    }
    CB200_REQUIRE(dtype_ != DType::Float16, "contiguous: float16 views are not supported");
    Tensor out(shape_, dtype_, stream_);
    cudeep_b200::StridedView view{};
    CB200_REQUIRE(ndim() <= cudeep_b200::StridedView::kMaxDims, "contiguous: rank above 8");
    view.ndim = static_cast<int>(ndim());
    for (int d = 0; d < view.ndim; ++d) {
        view.shape[d] = shape_[d];
        view.strides[d] = strides_[d];
    }
    if (numel() > 0) {
        if (dtype_ == DType::Float32)
            cudeep_b200::strided_copy<float>(static_cast<const float*>(data()), static_cast<float*>(out.data()),
                                             view, stream_);
        else
            cudeep_b200::strided_copy<double>(static_cast<const double*>(data()),
                                              static_cast<double*>(out.data()), view, stream_);
    }
    return out;
}

Tensor Tensor::binary(const Tensor& other, int op) const {
    CB200_REQUIRE(shape_ == other.shape_, "elementwise op: shape mismatch");
    CB200_REQUIRE(dtype_ == other.dtype_ && dtype_ != DType::Float16, "elementwise op: dtype mismatch");
    const Tensor a = contiguous(), b = other.contiguous();
    Tensor out(shape_, dtype_, stream_);
    const long long n = numel();
    if (n > 0) {
        long long blocks = (n + 255) / 256;
        if (blocks > 65535) blocks = 65535;
        if (dtype_ == DType::Float32)
            binary_kernel_f32<<<static_cast<unsigned>(blocks), 256, 0, stream_>>>(
                static_cast<const float*>(a.data()), static_cast<const float*>(b.data()),
                static_cast<float*>(out.data()), n, op);
        else
            binary_kernel_f64<<<static_cast<unsigned>(blocks), 256, 0, stream_>>>(
                static_cast<const double*>(a.data()), static_cast<const double*>(b.data()),
                static_cast<double*>(out.data()), n, op);
        CB200_CHECK_LAUNCH();
    }
    return out;
}

Tensor Tensor::operator+(const Tensor& other) const { return binary(other, 0); }
Tensor Tensor::operator-(const Tensor& other) const { return binary(other, 1); }
Tensor Tensor::operator*(const Tensor& other) const { return binary(other, 2); }

Tensor Tensor::matmul(const Tensor& other) const {
    CB200_REQUIRE(ndim() == 2 && other.ndim() == 2, "matmul requires 2-D tensors");
    CB200_REQUIRE(shape_[1] == other.shape_[0], "matmul: inner dimensions do not match");
    CB200_REQUIRE(dtype_ == other.dtype_, "matmul: dtype mismatch");
    CB200_REQUIRE(is_contiguous() && other.is_contiguous(), "matmul requires contiguous tensors");
    const int m = static_cast<int>(shape_[0]), k = static_cast<int>(shape_[1]);
    const int n = static_cast<int>(other.shape_[1]);
    Tensor out({shape_[0], other.shape_[1]}, dtype_, stream_);
    if (dtype_ == DType::Float32)
        kernels::launch_matmul_kernel<float>(static_cast<const float*>(data()),
                                             static_cast<const float*>(other.data()),
                                             static_cast<float*>(out.data()), m, n, k, stream_);
    else if (dtype_ == DType::Float64)
        kernels::launch_matmul_kernel<double>(static_cast<const double*>(data()),
                                              static_cast<const double*>(other.data()),
                                              static_cast<double*>(out.data()), m, n, k, stream_);
    else
        CB200_REQUIRE(false, "matmul: unsupported dtype");
    return out;
}

void Tensor::fill_(float value) {
    CB200_REQUIRE(is_contiguous(), "fill_: tensor must be contiguous");
    if (numel() == 0) return;
    if (dtype_ == DType::Float32)
        cudeep_b200::fill<float>(static_cast<float*>(data()), value, numel(), stream_);
    else if (dtype_ == DType::Float64)
        cudeep_b200::fill<double>(static_cast<double*>(data()), static_cast<double>(value), numel(), stream_);
    else
        CB200_REQUIRE(false, "fill_: unsupported dtype");
}

void Tensor::zero_() {
    if (numel() == 0) return;
    if (stream_) CB200_CUDA(cudaMemsetAsync(data(), 0, nbytes(), stream_));
    else CB200_CUDA(cudaMemset(data(), 0, nbytes()));
}

}  // namespace cudeep
