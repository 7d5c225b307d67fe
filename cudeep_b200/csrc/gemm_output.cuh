// FP32 row-major output of a GEMM tile, shared by the dense GEMM problem policies: bias and
// activation in registers, the register store paths (plain, and partial sums of a split tile),
// and the tensor map for bulk stores.  `Tile` needs m0 (first row of the CTA) and n0 (first column).
#pragma once

#include "epilogue_math.cuh"
#include "runtime.h"
#include "sm100_ptx.cuh"
#include "umma_gemm.cuh"

namespace cudeep_b200 {

struct GemmOutput {
    CUtensorMap map_c;     // C for bulk tensor stores: dims {N, M}, box {32, 32}, 128-byte swizzle
    float* c;
    long long ldc;
    int m, n;
    int vec_ok;            // rows of C are 16-byte aligned

    // Host: describes C; returns whether bulk tensor stores can be used (rows of 16-byte multiples).
    bool set_output(float* out, int rows, int cols, bool allow_bulk_store) {
        c = out;
        ldc = cols;
        m = rows;
        n = cols;
        vec_ok = ((cols % 4) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
        const bool bulk = vec_ok && allow_bulk_store;
        // Without bulk stores the map describes a dummy 32 x 32 view and is never used.
        const uint64_t dims[2] = {uint64_t(bulk ? cols : 32), uint64_t(bulk ? rows : 32)};
        const uint64_t strides[1] = {uint64_t(bulk ? cols : 32) * 4};
        const uint32_t box[2] = {32, 32};
        if (bulk) encode_tensor_map(&map_c, out, 2, dims, strides, box, TmaSwizzle::B128);
        else map_c = CUtensorMap{};
        return bulk;
    }

    __device__ __forceinline__ const CUtensorMap* out_map() const { return &map_c; }
    template <class Tile>
    __device__ __forceinline__ void out_coords(const Tile& t, int row_in_cta, int c0, int& x, int& y) const {
        x = t.n0 + c0;
        y = t.m0 + row_in_cta;
    }
    // Bias and activation of 32 columns of one row, in registers (the store clips what lies
    // outside C, so only the bias reads are bounded here).
    template <class Tile>
    __device__ __forceinline__ void finish(const Tile& t, int row_in_cta, int c0, float (&v)[32],
                                           const UmmaEpilogueArgs& epi) const {
        const int row = t.m0 + row_in_cta;
        const int col = t.n0 + c0;
        if (__builtin_expect(epi.bias != nullptr && row < m && col < n, 0)) {
            if (epi.bias_per_row) {
                const float b = __ldg(epi.bias + row);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += b;
            } else if (col + 32 <= n) {
                const float4* b4 = reinterpret_cast<const float4*>(epi.bias + col);
                if ((reinterpret_cast<uintptr_t>(b4) & 15u) == 0) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 b = __ldg(b4 + j);
                        v[4 * j] += b.x;
                        v[4 * j + 1] += b.y;
                        v[4 * j + 2] += b.z;
                        v[4 * j + 3] += b.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += __ldg(epi.bias + col + j);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col + j < n) v[j] += __ldg(epi.bias + col + j);
            }
        }
        apply_activation(v, epi.act);
    }

    template <class Tile>
    __device__ __forceinline__ void store(const Tile& t, int row_in_cta, int c0, float (&v)[32],
                                          const UmmaEpilogueArgs& epi, int mode) const {
        const int row = t.m0 + row_in_cta;
        const int col = t.n0 + c0;
        if (row >= m || col >= n) return;
        if (epi.bias != nullptr && mode != 2) {      // a split tile gets its bias once
            if (epi.bias_per_row) {
                const float b = __ldg(epi.bias + row);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += b;
            } else if (col + 32 <= n) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += __ldg(epi.bias + col + j);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col + j < n) v[j] += __ldg(epi.bias + col + j);
            }
        }
        float* dst = c + static_cast<long long>(row) * ldc + col;
        if (mode != 0) {
            // Partial sum of a split tile: C was zeroed before the launch and every K range
            // adds its share.  With two ranges the result does not depend on their order
            // (0 + p + q == 0 + q + p exactly); more ranges are summed in arrival order.
            if (vec_ok && col + 32 <= n) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    atomicAdd(reinterpret_cast<float4*>(dst + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col + j < n) atomicAdd(dst + j, v[j]);
            }
            return;
        }
        apply_activation(v, epi.act);
        if (vec_ok && col + 32 <= n) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col + j < n) dst[j] = v[j];
        }
    }
};

}  // namespace cudeep_b200
