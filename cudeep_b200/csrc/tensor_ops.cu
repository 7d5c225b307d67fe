// Small data-movement kernels behind the Tensor host type: strided copy
// (materialising a transposed / reshaped view), fill, broadcast row add and the
// standalone activations.  All are one pass over the data (HBM-bound).
//
// strided_copy replaces the reference's launch_strided_copy (src/tensor.cu:47-68),
// which allocates two device arrays, copies shape and strides to them and
// synchronises the stream on every call; here shape and strides travel as kernel
// arguments and nothing blocks.
#include "tensor_ops.h"
#include "epilogue_math.cuh"

namespace cudeep_b200 {

namespace {

template <typename T>
__global__ void strided_copy_kernel(const T* __restrict__ src, T* __restrict__ dst, StridedView view,
                                    long long total) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        long long rest = i, offset = 0;
#pragma unroll 1
        for (int d = view.ndim - 1; d >= 0; --d) {
            const long long idx = rest % view.shape[d];
            rest /= view.shape[d];
            offset += idx * view.strides[d];
        }
        dst[i] = src[offset];
    }
}

// 2-D transpose through shared memory: dst[c][r] = src[r][c]; both sides coalesced.
template <typename T>
__global__ void transpose2d_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows, int cols) {
    __shared__ T tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[i][threadIdx.x] = src[static_cast<long long>(r) * cols + c];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (r < rows && c < cols) dst[static_cast<long long>(c) * rows + r] = tile[threadIdx.x][i];
    }
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ dst, T value, long long total) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        dst[i] = value;
}

template <typename T>
__global__ void add_row_kernel(const T* __restrict__ m, const T* __restrict__ row, T* __restrict__ out,
                               long long total, int cols) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = m[i] + row[i % cols];
}

__global__ void activation_kernel(const float* __restrict__ x, float* __restrict__ y, long long total, int act) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        y[i] = apply_activation1(x[i], act);
}

unsigned grid_for(long long total) {
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(device_info().num_sms) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

}  // namespace

template <typename T>
void strided_copy(const T* src, T* dst, const StridedView& view, cudaStream_t stream) {
    CB200_REQUIRE(view.ndim >= 1 && view.ndim <= StridedView::kMaxDims, "strided copy: rank must be 1..8");
    long long total = 1;
    for (int d = 0; d < view.ndim; ++d) {
        CB200_REQUIRE(view.shape[d] > 0, "strided copy: extents must be positive");
        total *= view.shape[d];
    }
    // The common case, a transposed matrix, takes the tiled transpose.
    if (view.ndim == 2 && view.strides[0] == 1 && view.strides[1] == view.shape[0]) {
        const int rows = static_cast<int>(view.shape[1]), cols = static_cast<int>(view.shape[0]);
        dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
        if (grid.y <= 65535) {
            transpose2d_kernel<T><<<grid, block, 0, stream>>>(src, dst, rows, cols);
            CB200_CHECK_LAUNCH();
            return;
        }
    }
    strided_copy_kernel<T><<<grid_for(total), 256, 0, stream>>>(src, dst, view, total);
    CB200_CHECK_LAUNCH();
}
template void strided_copy<float>(const float*, float*, const StridedView&, cudaStream_t);
template void strided_copy<double>(const double*, double*, const StridedView&, cudaStream_t);

template <typename T>
void fill(T* dst, T value, long long total, cudaStream_t stream) {
    if (total <= 0) return;
    fill_kernel<T><<<grid_for(total), 256, 0, stream>>>(dst, value, total);
    CB200_CHECK_LAUNCH();
}
template void fill<float>(float*, float, long long, cudaStream_t);
template void fill<double>(double*, double, long long, cudaStream_t);

template <typename T>
void add_row(const T* m, const T* row, T* out, long long rows, int cols, cudaStream_t stream) {
    CB200_REQUIRE(rows > 0 && cols > 0, "broadcast add: extents must be positive");
    add_row_kernel<T><<<grid_for(rows * cols), 256, 0, stream>>>(m, row, out, rows * cols, cols);
    CB200_CHECK_LAUNCH();
}
template void add_row<float>(const float*, const float*, float*, long long, int, cudaStream_t);
template void add_row<double>(const double*, const double*, double*, long long, int, cudaStream_t);

void activation(const float* x, float* y, long long total, int act, cudaStream_t stream) {
    CB200_REQUIRE(act >= 0 && act <= 4, "unknown activation code");
    if (total <= 0) return;
    activation_kernel<<<grid_for(total), 256, 0, stream>>>(x, y, total, act);
    CB200_CHECK_LAUNCH();
}

}  // namespace cudeep_b200
