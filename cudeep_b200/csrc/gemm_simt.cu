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

#include <cuda_bf16.h>
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
template <> __device__ __forceinline__ float widen<float, __nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

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
// 16-byte aligned.  K slices of 16 travel global -> shared memory with cp.async, STAGES - 1
// slices in flight while one is multiplied, so global latency hides behind the FMAs even
// when only a few warps fit on an SM (512^3 gives each SM one small CTA).  A stays row-major
// in shared memory ([BM][16 + 4]); a thread reads 4 consecutive k of a row with one 128-bit
// load, and all threads of a warp that share a row read the same address (broadcast).
// B is [K,N].  Sums run in ascending k.
template <int BM, int BN, int TM, int TN, int STAGES>
__global__ void __launch_bounds__((BM / TM) * (BN / TN), 2)
sgemm_aligned_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                     int m, int n, int k, const float* __restrict__ bias, int bias_per_row, int act) {
    constexpr int BK = 16;
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int A_LD = BK + 4;                 // floats per shared-memory row of A
    constexpr int B_LD = BN + 4;
    constexpr int A_CHUNKS = BM * BK / 4;        // 16-byte copies per slice
    constexpr int B_CHUNKS = BK * BN / 4;
    static_assert(TM % 4 == 0 && TN % 4 == 0, "micro-tile must be a multiple of 4");
    extern __shared__ __align__(16) float smem_f[];
    float* as = smem_f;                                   // [STAGES][BM][A_LD]
    float* bs = smem_f + STAGES * BM * A_LD;              // [STAGES][BK][B_LD]

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const float* a_tile = a + static_cast<long long>(blockIdx.y) * BM * k;
    const float* b_tile = b + static_cast<long long>(blockIdx.x) * BN;

    auto issue = [&](int slice, int buf) {
        const int k0 = slice * BK;
        for (int v = tid; v < A_CHUNKS; v += THREADS) {
            const int row = v / (BK / 4), kq = (v % (BK / 4)) * 4;
            const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(as + (buf * BM + row) * A_LD + kq));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                         "l"(a_tile + static_cast<long long>(row) * k + k0 + kq));
        }
        for (int v = tid; v < B_CHUNKS; v += THREADS) {
            const int kk = v / (BN / 4), nq = (v % (BN / 4)) * 4;
            const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(bs + (buf * BK + kk) * B_LD + nq));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                         "l"(b_tile + static_cast<long long>(k0 + kk) * n + nq));
        }
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    const int slices = k / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < slices) issue(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int s = 0; s < slices; ++s) {
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();                      // slice s has landed; buffer (s - 1) % STAGES is free again
        if (s + STAGES - 1 < slices) issue(s + STAGES - 1, (s + STAGES - 1) % STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const float* as_s = as + (s % STAGES) * BM * A_LD;
        const float* bs_s = bs + (s % STAGES) * BK * B_LD;
#pragma unroll
        for (int k4 = 0; k4 < BK; k4 += 4) {
            float4 av[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i)
                av[i] = *reinterpret_cast<const float4*>(as_s + (ty * TM + i) * A_LD + k4);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                float bv[TN];
#pragma unroll
                for (int j = 0; j < TN; j += 4)
                    *reinterpret_cast<float4*>(&bv[j]) =
                        *reinterpret_cast<const float4*>(bs_s + (k4 + kk) * B_LD + tx * TN + j);
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float ai = kk == 0 ? av[i].x : kk == 1 ? av[i].y : kk == 2 ? av[i].z : av[i].w;
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ai, bv[j], acc[i][j]);
                }
            }
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

template <int BM, int BN, int TM, int TN, int STAGES>
void launch_aligned(const float* a, const float* b, float* c, int m, int n, int k, const float* bias,
                    bool bias_per_row, int act, cudaStream_t stream) {
    constexpr size_t smem = sizeof(float) * STAGES * (BM * (16 + 4) + 16 * (BN + 4));
    auto kernel = sgemm_aligned_kernel<BM, BN, TM, TN, STAGES>;
    ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    dim3 grid(n / BN, m / BM);
    CB200_TRACE("gemm strict FP32 (cp.async, aligned): M=%d N=%d K=%d tile=%dx%d stages=%d grid=%ux%u", m, n, k, BM,
                BN, STAGES, grid.x, grid.y);
    kernel<<<grid, (BM / TM) * (BN / TN), smem, stream>>>(a, b, c, m, n, k, bias, bias_per_row ? 1 : 0, act);
    CB200_CHECK_LAUNCH();
}

template <typename TI, typename T, int BM, int BN, int BK, int TM, int TN>
void launch(const TI* a, const TI* b, bool b_is_nk, T* c, int m, int n, int k, const T* bias,
            bool bias_per_row, int act, cudaStream_t stream) {
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    dim3 block((BM / TM) * (BN / TN));
    CB200_TRACE("gemm strict %s (SIMT, any shape): M=%d N=%d K=%d B=%s tile=%dx%d grid=%ux%u",
                sizeof(T) == 8 ? "FP64" : "FP32", m, n, k, b_is_nk ? "[N,K]" : "[K,N]", BM, BN, grid.x, grid.y);
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
            launch_aligned<128, 128, 8, 8, 3>(a, b, c, m, n, k, bias, bias_per_row, act, stream);
            return;
        }
        if (m % 64 == 0 && n % 64 == 0 && static_cast<long long>(m / 64) * (n / 64) >= sms) {
            launch_aligned<64, 64, 4, 4, 4>(a, b, c, m, n, k, bias, bias_per_row, act, stream);
            return;
        }
        if (m % 32 == 0 && n % 64 == 0) {
            launch_aligned<32, 64, 4, 4, 4>(a, b, c, m, n, k, bias, bias_per_row, act, stream);
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

void gemm_simt_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, float* c, int m, int n, int k,
                    cudaStream_t stream) {
    CB200_REQUIRE(m > 0 && n > 0 && k > 0, "GEMM extents must be positive");
    launch<__nv_bfloat16, float, 64, 64, 16, 4, 4>(a, b, false, c, m, n, k, nullptr, false, EPI_NONE, stream);
}

}  // namespace cudeep_b200
