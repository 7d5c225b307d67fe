// FP16 GEMM on tcgen05 behind launch_matmul_kernel_fp16 (reference include/cudeep/kernels/
// matmul.cuh:27-30, src/kernels/matmul_kernel.cu:755-930: half A[M,K], half B[K,N], float C).
//
// The mainloop is the TF32 kernel's with kind::f16 MMAs: a K block is 64 halves = the same 128
// bytes per operand row, so tiles, stages, barriers, the TMEM accumulators and the epilogue are
// shared.  A is K-major; B[K,N] is MN-major and is staged as 64-column x 64-row TMA boxes in the
// plain 128-byte swizzle (16-bit MN-major operands need no special swizzle atom, unlike 32-bit).
#include "gemm_f16.h"
#include "gemm_output.cuh"
#include "umma_gemm.cuh"

namespace cudeep_b200 {

namespace {

constexpr int F16_BK = 64;      // halves per K block
constexpr int F16_CHUNK = 64;   // B columns per 128-byte row of a box

template <int CTAS, int BN>
struct GemmProblemF16 : GemmOutput {
    static constexpr bool kTmaStore = true;
    static constexpr bool kClusterSplit = false;
    CUtensorMap map_a;     // dims {K, M}, box {64, 128}
    CUtensorMap map_b;     // chunked: dims {64, K, N/64}, box {64, 64, chunks per CTA}; else dims {N, K}, box {64, 64}
    int b_chunked;

    struct Tile {
        int m0, n0, nb0;
    };

    __device__ __forceinline__ void prefetch_maps() const {
        ptx::prefetch_tensormap(&map_a);
        ptx::prefetch_tensormap(&map_b);
        ptx::prefetch_tensormap(&map_c);
    }
    __device__ __forceinline__ Tile decode(int tm, int tn, uint32_t cta_rank) const {
        Tile t;
        t.m0 = (tm * CTAS + int(cta_rank)) * UMMA_BM;
        t.n0 = tn * BN;
        t.nb0 = t.n0 + int(cta_rank) * (BN / CTAS);
        return t;
    }
    template <int C>
    __device__ __forceinline__ void load(const Tile& t, int kb, uint32_t a_smem, uint32_t b_smem,
                                         uint32_t bar) const {
        const int k0 = kb * F16_BK;
        if constexpr (C == 1) {
            ptx::tma_load_2d(a_smem, &map_a, bar, k0, t.m0);
            if (b_chunked) {
                ptx::tma_load_3d(b_smem, &map_b, bar, 0, k0, t.nb0 / F16_CHUNK);
            } else {
#pragma unroll
                for (int j = 0; j < BN / CTAS / F16_CHUNK; ++j)
                    ptx::tma_load_2d(b_smem + j * 8192, &map_b, bar, t.nb0 + j * F16_CHUNK, k0);
            }
        } else {
            ptx::tma_load_2d_pair(a_smem, &map_a, bar, k0, t.m0);
            if (b_chunked) {
                ptx::tma_load_3d_pair(b_smem, &map_b, bar, 0, k0, t.nb0 / F16_CHUNK);
            } else {
#pragma unroll
                for (int j = 0; j < BN / CTAS / F16_CHUNK; ++j)
                    ptx::tma_load_2d_pair(b_smem + j * 8192, &map_b, bar, t.nb0 + j * F16_CHUNK, k0);
            }
        }
    }
};

// KIND: UMMA_KIND_F16 or UMMA_KIND_BF16; the operands are 2-byte words either way (the tensor maps
// only move them), the MMA's instruction descriptor says how to read them.
template <int CTAS, int KATOMS, int KIND = UMMA_KIND_F16>
void launch_f16(const void* a, const void* b, float* c, int m, int n, int k, uint32_t b_lbo, uint32_t b_sbo,
                cudaStream_t stream) {
    constexpr int BN = 256;
    using Cfg = UmmaConfig<CTAS, BN, true, KATOMS>;
    using Prob = GemmProblemF16<CTAS, BN>;
    const DeviceInfo& dev = device_info();

    Prob prob;
    {
        const uint64_t dims[2] = {uint64_t(k), uint64_t(m)};
        const uint64_t strides[1] = {uint64_t(k) * 2};
        const uint32_t box[2] = {F16_BK, UMMA_BM};
        encode_tensor_map_f16(&prob.map_a, a, 2, dims, strides, box, TmaSwizzle::B128);
    }
    prob.b_chunked = (n % F16_CHUNK == 0) ? 1 : 0;
    if (prob.b_chunked) {
        const uint64_t dims[3] = {F16_CHUNK, uint64_t(k), uint64_t(n / F16_CHUNK)};
        const uint64_t strides[2] = {uint64_t(n) * 2, 128};
        const uint32_t box[3] = {F16_CHUNK, F16_BK, uint32_t(Cfg::BN_CTA / F16_CHUNK)};
        encode_tensor_map_f16(&prob.map_b, b, 3, dims, strides, box, TmaSwizzle::B128);
    } else {
        const uint64_t dims[2] = {uint64_t(n), uint64_t(k)};
        const uint64_t strides[1] = {uint64_t(n) * 2};
        const uint32_t box[2] = {F16_CHUNK, F16_BK};
        encode_tensor_map_f16(&prob.map_b, b, 2, dims, strides, box, TmaSwizzle::B128);
    }
    const bool tma_store = prob.set_output(c, m, n, true);

    const uint32_t staging_bytes = tma_store ? UMMA_STORE_STAGING_BYTES : 0u;
    const int fit_stages = int((Cfg::SMEM_BUDGET - staging_bytes) / Cfg::STAGE_BYTES);
    UmmaSchedule sched = whole_tile_schedule((m + UMMA_BM * CTAS - 1) / (UMMA_BM * CTAS), (n + BN - 1) / BN,
                                             (k + F16_BK - 1) / F16_BK, BN, Cfg::TX_BYTES,
                                             fit_stages < Cfg::STAGES ? fit_stages : Cfg::STAGES, dev.status_word);
    sched.b_lbo = b_lbo;
    sched.b_sbo = b_sbo;
    sched.tma_store = tma_store ? 1 : 0;
    sched.ring_staging = uint32_t(sched.stages) * Cfg::STAGE_BYTES >= 131072u ? 1 : 0;
    const uint32_t smem_bytes = uint32_t(sched.stages) * Cfg::STAGE_BYTES + staging_bytes + 1024;

    const long long num_tiles = static_cast<long long>(sched.tiles_m) * sched.tiles_n;
    long long groups = dev.num_sms / CTAS;
    if (groups < 1) groups = 1;
    if (groups > num_tiles) groups = num_tiles;

    CB200_TRACE("gemm %s tcgen05: M=%d N=%d K=%d tile=%dx%d ctas/mma=%d stages=%d clusters=%lld store=%s",
                KIND == UMMA_KIND_BF16 ? "bf16" : "f16", m, n, k, UMMA_BM * CTAS, BN, CTAS, sched.stages, groups, tma_store ? "bulk-tensor" : "registers");
    auto kernel = umma_tf32_kernel<CTAS, BN, true, KATOMS, Prob, false, KIND>;
    UmmaEpilogueArgs epi{nullptr, 0, EPI_NONE};
    launch_umma(kernel, prob, sched, epi, groups, CTAS, smem_bytes, Cfg::SMEM_MAX, stream);
}

}  // namespace

bool gemm_f16_supported(const void* a, const void* b, int m, int n, int k) {
    if (m < 64 || n < 64 || k < 64) return false;
    if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u)) return false;
    if (k % 8 != 0 || n % 8 != 0) return false;
    return device_info().cc_major == 10;
}

void gemm_f16(const __half* a, const __half* b, float* c, int m, int n, int k, int ctas, uint32_t b_lbo,
              uint32_t b_sbo, cudaStream_t stream) {
    CB200_REQUIRE(gemm_f16_supported(a, b, m, n, k),
                  "FP16 tensor-core GEMM needs an sm_100 device, 16-byte aligned operands, K and N multiples "
                  "of 8 and M, N, K of at least 64");
    if (ctas == 0) {
        const long long pair_tiles = static_cast<long long>((m + 255) / 256) * ((n + 255) / 256);
        ctas = pair_tiles * 2 >= device_info().num_sms / 2 ? 2 : 1;
    }
    if (ctas == 2) launch_f16<2, 2>(a, b, c, m, n, k, b_lbo, b_sbo, stream);
    else launch_f16<1, 1>(a, b, c, m, n, k, b_lbo, b_sbo, stream);
}

void gemm_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, float* c, int m, int n, int k, int ctas,
               cudaStream_t stream) {
    CB200_REQUIRE(gemm_f16_supported(a, b, m, n, k),
                  "BF16 tensor-core GEMM needs an sm_100 device, 16-byte aligned operands, K and N multiples "
                  "of 8 and M, N, K of at least 64");
    if (ctas == 0) {
        const long long pair_tiles = static_cast<long long>((m + 255) / 256) * ((n + 255) / 256);
        ctas = pair_tiles * 2 >= device_info().num_sms / 2 ? 2 : 1;
    }
    if (ctas == 2) launch_f16<2, 2, UMMA_KIND_BF16>(a, b, c, m, n, k, 0, 0, stream);
    else launch_f16<1, 1, UMMA_KIND_BF16>(a, b, c, m, n, k, 0, 0, stream);
}

}  // namespace cudeep_b200
