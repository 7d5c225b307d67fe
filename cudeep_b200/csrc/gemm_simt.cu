// Strict-precision SIMT GEMM: the path for callers that need exact FP32
// (reference launch_matmul_kernel_fp32, src/kernels/matmul_kernel.cu:1851-1863),
// for FP64 (launch_matmul_kernel<double>, :1843-1849) and for shapes the
// tensor-core path does not take (tiny or unaligned problems).
//
// Each CTA computes a BM x BN tile; K is walked in BK slices staged in shared
// memory (A transposed so the inner loop reads both operands conflict-free).
// Every thread accumulates a TM x TN micro-tile with fused multiply-adds in
// ascending-k order, so results do not depend on the grid shape.
#include "gemm_simt.h"
#include "epilogue_math.cuh"

#include <cuda_fp16.h>

namespace cudeep_b200 {

namespace {

template <typename T> __device__ __forceinline__ T fma_t(T a, T b, T c);
template <> __device__ __forceinline__ float fma_t<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double fma_t<double>(double a, double b, double c) { return fma(a, b, c); }

template <typename T> __device__ __forceinline__ T act_t(T x, int act);
template <> __device__ __forceinline__ float act_t<float>(float x, int act) { return apply_activation1(x, act); }
template <> __device__ __forceinline__ double act_t<double>(double x, int act) {
    switch (act) {
        case EPI_RELU: return x > 0.0 ? x : 0.0;
        case EPI_GELU: return 0.5 * x * (1.0 + tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)));
        case EPI_SILU: return x / (1.0 + exp(-x));
        case EPI_SIGMOID: return 1.0 / (1.0 + exp(-x));
        default: return x;
    }
}

template <typename T, typename TI> __device__ __forceinline__ T widen(TI x) { return static_cast<T>(x); }
template <> __device__ __forceinline__ float widen<float, __half>(__half x) { return __half2float(x); }

// TI: element type of A and B in memory; T: accumulate / output type.
template <typename TI, typename T, int BM, int BN, int BK, int TM, int TN, bool B_NK, bool A_KM = false>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const TI* __restrict__ a, const TI* __restrict__ b, T* __restrict__ c, int m, int n,
                 int k, const T* __restrict__ bias, int bias_per_row, int act) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ T as[BK][BM + 4];
    __shared__ T bs[BK][BN + 4];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const long long m0 = static_cast<long long>(blockIdx.y) * BM;
    const long long n0 = static_cast<long long>(blockIdx.x) * BN;

    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = T(0);

    for (int k0 = 0; k0 < k; k0 += BK) {
        // A tile: BM rows x BK columns, read along K (contiguous), stored transposed.
        for (int idx = tid; idx < BM * BK; idx += THREADS) {
            const int r = idx / BK, kk = idx % BK;
            const long long gr = m0 + r;
            const int gk = k0 + kk;
            as[kk][r] = (gr < m && gk < k)
                            ? widen<T, TI>(A_KM ? a[static_cast<long long>(gk) * m + gr] : a[gr * k + gk])
                            : T(0);
        }
        if (B_NK) {
            for (int idx = tid; idx < BN * BK; idx += THREADS) {
                const int col = idx / BK, kk = idx % BK;
                const long long gc = n0 + col;
                const int gk = k0 + kk;
                bs[kk][col] = (gc < n && gk < k) ? widen<T, TI>(b[gc * k + gk]) : T(0);
            }
        } else {
            for (int idx = tid; idx < BN * BK; idx += THREADS) {
                const int kk = idx / BN, col = idx % BN;
                const long long gc = n0 + col;
                const int gk = k0 + kk;
                bs[kk][col] = (gc < n && gk < k) ? widen<T, TI>(b[static_cast<long long>(gk) * n + gc]) : T(0);
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            T ra[TM], rb[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ra[i] = as[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) rb[j] = bs[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fma_t<T>(ra[i], rb[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long gr = m0 + ty * TM + i;
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const long long gc = n0 + tx * TN + j;
            if (gc >= n) continue;
            T v = acc[i][j];
            if (bias != nullptr) v += bias_per_row ? bias[gr] : bias[gc];
            c[gr * n + gc] = act_t<T>(v, act);
        }
    }
}

// Fast path for FP32 when every extent is a multiple of the tile and the operands are
// 16-byte aligned: 128-bit global loads, the next K slice prefetched into registers
// while the current one is multiplied out of shared memory (two buffers, one barrier
// per slice), 128-bit shared-memory reads in the inner loop.  B is [K,N].
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_aligned_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                     int m, int n, int k, const float* __restrict__ bias, int bias_per_row, int act) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int A_VEC = BM * BK / 4 / THREADS;     // float4 loads of A per thread and slice
    constexpr int B_VEC = BK * BN / 4 / THREADS;
    static_assert(A_VEC >= 1 && B_VEC >= 1 && TM % 4 == 0 && TN % 4 == 0 && BK % 4 == 0, "tile shape");
    __shared__ __align__(16) float as[2][BK][BM + 4];
    __shared__ __align__(16) float bs[2][BK][BN + 4];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const float* a_tile = a + static_cast<long long>(blockIdx.y) * BM * k;
    const float* b_tile = b + static_cast<long long>(blockIdx.x) * BN;

    float4 ra[A_VEC], rb[B_VEC];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < A_VEC; ++i) {
            const int v = tid + i * THREADS;
            const int row = v / (BK / 4), kq = (v % (BK / 4)) * 4;
            ra[i] = *reinterpret_cast<const float4*>(a_tile + static_cast<long long>(row) * k + k0 + kq);
        }
#pragma unroll
        for (int i = 0; i < B_VEC; ++i) {
            const int v = tid + i * THREADS;
            const int kk = v / (BN / 4), nq = (v % (BN / 4)) * 4;
            rb[i] = *reinterpret_cast<const float4*>(b_tile + static_cast<long long>(k0 + kk) * n + nq);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_VEC; ++i) {
            const int v = tid + i * THREADS;
            const int row = v / (BK / 4), kq = (v % (BK / 4)) * 4;
            as[buf][kq + 0][row] = ra[i].x;
            as[buf][kq + 1][row] = ra[i].y;
            as[buf][kq + 2][row] = ra[i].z;
            as[buf][kq + 3][row] = ra[i].w;
        }
#pragma unroll
        for (int i = 0; i < B_VEC; ++i) {
            const int v = tid + i * THREADS;
            const int kk = v / (BN / 4), nq = (v % (BN / 4)) * 4;
            *reinterpret_cast<float4*>(&bs[buf][kk][nq]) = rb[i];
        }
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    fetch(0);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = 0; k0 < k; k0 += BK) {
        const bool more = k0 + BK < k;
        if (more) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], bv[TN];
#pragma unroll
            for (int i = 0; i < TM; i += 4)
                *reinterpret_cast<float4*>(&av[i]) = *reinterpret_cast<const float4*>(&as[buf][kk][ty * TM + i]);
#pragma unroll
            for (int j = 0; j < TN; j += 4)
                *reinterpret_cast<float4*>(&bv[j]) = *reinterpret_cast<const float4*>(&bs[buf][kk][tx * TN + j]);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (more) {
            stash(buf ^ 1);
            __syncthreads();
            buf ^= 1;
        }
    }

    const long long row0 = static_cast<long long>(blockIdx.y) * BM + ty * TM;
    const long long col0 = static_cast<long long>(blockIdx.x) * BN + tx * TN;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
#pragma unroll
        for (int j = 0; j < TN; j += 4) {
            float v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float x = acc[i][j + q];
                if (bias != nullptr) x += bias_per_row ? bias[row0 + i] : bias[col0 + j + q];
                v[q] = apply_activation1(x, act);
            }
            *reinterpret_cast<float4*>(c + (row0 + i) * n + col0 + j) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
}

template <int BM, int BN, int BK, int TM, int TN>
void launch_aligned(const float* a, const float* b, float* c, int m, int n, int k, const float* bias,
                    bool bias_per_row, int act, cudaStream_t stream) {
    dim3 grid(n / BN, m / BM);
    sgemm_aligned_kernel<BM, BN, BK, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, stream>>>(
        a, b, c, m, n, k, bias, bias_per_row ? 1 : 0, act);
    CB200_CHECK_LAUNCH();
}

template <typename TI, typename T, int BM, int BN, int BK, int TM, int TN>
void launch(const TI* a, const TI* b, bool b_is_nk, T* c, int m, int n, int k, const T* bias,
            bool bias_per_row, int act, cudaStream_t stream) {
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    dim3 block((BM / TM) * (BN / TN));
    if (b_is_nk)
        gemm_simt_kernel<TI, T, BM, BN, BK, TM, TN, true><<<grid, block, 0, stream>>>(
            a, b, c, m, n, k, bias, bias_per_row ? 1 : 0, act);
    else
        gemm_simt_kernel<TI, T, BM, BN, BK, TM, TN, false><<<grid, block, 0, stream>>>(
            a, b, c, m, n, k, bias, bias_per_row ? 1 : 0, act);
    CB200_CHECK_LAUNCH();
}

}  // namespace

template <>
void gemm_simt<float>(const float* a, const float* b, bool b_is_nk, float* c, int m, int n, int k,
                      const float* bias, bool bias_per_row, int act, cudaStream_t stream) {
    CB200_REQUIRE(m > 0 && n > 0 && k > 0, "GEMM extents must be positive");
    const long long big_tiles = static_cast<long long>((m + 127) / 128) * ((n + 127) / 128);
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                             reinterpret_cast<uintptr_t>(c)) & 15u) == 0;
    if (!b_is_nk && aligned16 && k % 16 == 0) {
        const long long sms = device_info().num_sms;
        if (m % 128 == 0 && n % 128 == 0 && big_tiles >= sms) {
            launch_aligned<128, 128, 16, 8, 8>(a, b, c, m, n, k, bias, bias_per_row, act, stream);
            return;
        }
        if (m % 64 == 0 && n % 64 == 0 && static_cast<long long>(m / 64) * (n / 64) >= sms) {
            launch_aligned<64, 64, 16, 4, 4>(a, b, c, m, n, k, bias, bias_per_row, act, stream);
            return;
        }
        if (m % 32 == 0 && n % 64 == 0) {
            launch_aligned<32, 64, 16, 4, 4>(a, b, c, m, n, k, bias, bias_per_row, act, stream);
            return;
        }
    }
    if (big_tiles >= 2LL * device_info().num_sms)
        launch<float, float, 128, 128, 16, 8, 8>(a, b, b_is_nk, c, m, n, k, bias, bias_per_row, act, stream);
    else
        launch<float, float, 64, 64, 16, 4, 4>(a, b, b_is_nk, c, m, n, k, bias, bias_per_row, act, stream);
}

template <>
void gemm_simt<double>(const double* a, const double* b, bool b_is_nk, double* c, int m, int n,
                       int k, const double* bias, bool bias_per_row, int act, cudaStream_t stream) {
    CB200_REQUIRE(m > 0 && n > 0 && k > 0, "GEMM extents must be positive");
    launch<double, double, 64, 64, 16, 4, 4>(a, b, b_is_nk, c, m, n, k, bias, bias_per_row, act, stream);
}

void gemm_simt_tn(const float* a, const float* b, float* c, int m, int n, int k, cudaStream_t stream) {
    CB200_REQUIRE(m > 0 && n > 0 && k > 0, "GEMM extents must be positive");
    dim3 grid((n + 63) / 64, (m + 63) / 64);
    gemm_simt_kernel<float, float, 64, 64, 16, 4, 4, false, true><<<grid, 256, 0, stream>>>(
        a, b, c, m, n, k, nullptr, 0, EPI_NONE);
    CB200_CHECK_LAUNCH();
}

void gemm_simt_half(const __half* a, const __half* b, float* c, int m, int n, int k,
                    cudaStream_t stream) {
    CB200_REQUIRE(m > 0 && n > 0 && k > 0, "GEMM extents must be positive");
    launch<__half, float, 64, 64, 16, 4, 4>(a, b, false, c, m, n, k, nullptr, false, EPI_NONE, stream);
}

}  // namespace cudeep_b200
