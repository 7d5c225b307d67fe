// Dense TF32 GEMM on tcgen05: C[M,N] = act(A[M,K] * B + bias).
//
// Two B layouts share one kernel:
//   * B[K,N] row-major (the layout of Tensor.matmul, reference
//     src/tensor.cu:384-420 / matmul_kernel.cu:1785-1841): an MN-major UMMA
//     operand, staged as 32-column x 32-row TMA boxes in the 128-byte swizzle
//     with 32-byte atoms (the one layout tcgen05 takes for MN-major 32-bit data).
//   * W[N,K] row-major (nn.Linear's weight as stored, reference
//     python/cuDeep/nn.py:110-115): a K-major operand, so Linear needs no
//     transposed copy of W.
// Operands are read as raw FP32 words; the tensor core ignores the low 13
// mantissa bits, the same truncation the reference's mma.sync path applies
// (matmul_kernel.cu:186-201).
#include "gemm_tf32.h"
#include "gemm_output.cuh"
#include "umma_gemm.cuh"

#include <type_traits>

namespace cudeep_b200 {

namespace {

template <int CTAS, int BN, bool B_MN_MAJOR, bool A_MN_MAJOR = false>
struct GemmProblem : GemmOutput {
    CUtensorMap map_a;     // K-major: dims {K, M}, box {32, 128};  MN-major (A stored [K, M]): as map_b
    CUtensorMap map_b;     // K-major: dims {K, N}, box {32, BN/CTAS};  MN-major: dims {N, K}, box {32, 32}
    int b_chunked;         // MN-major B described as {32, K, N/32}: one load brings every column chunk
    int a_chunked;         // the same for an MN-major A

    static constexpr bool kTmaStore = true;
    static constexpr bool kClusterSplit = true;

    struct Tile {
        int m0;            // first C row of this CTA
        int n0;            // first C column of the tile
        int nb0;           // first B row (K-major) / column (MN-major) this CTA stages
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
        const int k0 = kb * UMMA_BK;
        if constexpr (C == 1) {
            if constexpr (A_MN_MAJOR) {
                if (a_chunked) {
                    ptx::tma_load_3d(a_smem, &map_a, bar, 0, k0, t.m0 / 32);
                } else {
#pragma unroll
                    for (int j = 0; j < UMMA_BM / 32; ++j)
                        ptx::tma_load_2d(a_smem + j * 4096, &map_a, bar, t.m0 + j * 32, k0);
                }
            } else {
                ptx::tma_load_2d(a_smem, &map_a, bar, k0, t.m0);
            }
            if constexpr (B_MN_MAJOR) {
                if (b_chunked) {
                    ptx::tma_load_3d(b_smem, &map_b, bar, 0, k0, t.nb0 / 32);
                } else {
#pragma unroll
                    for (int j = 0; j < BN / CTAS / 32; ++j)
                        ptx::tma_load_2d(b_smem + j * 4096, &map_b, bar, t.nb0 + j * 32, k0);
                }
            } else {
                ptx::tma_load_2d(b_smem, &map_b, bar, k0, t.nb0);
            }
        } else {
            if constexpr (A_MN_MAJOR) {
                if (a_chunked) {
                    ptx::tma_load_3d_pair(a_smem, &map_a, bar, 0, k0, t.m0 / 32);
                } else {
#pragma unroll
                    for (int j = 0; j < UMMA_BM / 32; ++j)
                        ptx::tma_load_2d_pair(a_smem + j * 4096, &map_a, bar, t.m0 + j * 32, k0);
                }
            } else {
                ptx::tma_load_2d_pair(a_smem, &map_a, bar, k0, t.m0);
            }
            if constexpr (B_MN_MAJOR) {
                if (b_chunked) {
                    ptx::tma_load_3d_pair(b_smem, &map_b, bar, 0, k0, t.nb0 / 32);
                } else {
#pragma unroll
                    for (int j = 0; j < BN / CTAS / 32; ++j)
                        ptx::tma_load_2d_pair(b_smem + j * 4096, &map_b, bar, t.nb0 + j * 32, k0);
                }
            } else {
                ptx::tma_load_2d_pair(b_smem, &map_b, bar, k0, t.nb0);
            }
        }
    }
};

// The same problem for one rank of a row-sharded product whose result every rank wants whole: each
// staged 32 x 32 block is stored into this GPU's C and into the same place of the other ranks' C
// (tensor maps over peer-mapped device memory).  Bulk stores only; nothing is loaded from a peer.
template <int CTAS, int BN, bool B_MN_MAJOR>
struct GemmPushProblem : GemmProblem<CTAS, BN, B_MN_MAJOR, false> {
    static constexpr bool kPeerStore = true;
    static constexpr bool kClusterSplit = false;       // every tile is whole: partial sums are never pushed
    CUtensorMap peer_c[kMaxGemmPeers];
    int n_peers;

    __device__ __forceinline__ void prefetch_maps() const {
        GemmProblem<CTAS, BN, B_MN_MAJOR, false>::prefetch_maps();
        for (int i = 0; i < n_peers; ++i) ptx::prefetch_tensormap(&peer_c[i]);
    }
    __device__ __forceinline__ void push(uint32_t block, int x, int y) const {
        for (int i = 0; i < n_peers; ++i) ptx::tma_store_2d(&peer_c[i], block, x, y);
    }
};

// And the form for GPUs behind one NVSwitch: `mc_c` is this rank's rows of C seen through a multicast
// address, so one multimem.st per 16 bytes writes them into every GPU's C (this GPU's included).  The
// rank then sends each tile over NVLink once, whatever the number of peers.
template <int CTAS, int BN, bool B_MN_MAJOR>
struct GemmMultimemProblem : GemmProblem<CTAS, BN, B_MN_MAJOR, false> {
    static constexpr bool kMultimemStore = true;
    static constexpr bool kClusterSplit = false;
    float* mc_c;

    // Rows [y, y + 32), columns [x, x + 32) of this rank's C from the staged block (128-byte rows,
    // 16-byte units XOR-swizzled by row): each instruction of the warp covers four rows.
    __device__ __forceinline__ void multimem_store(uint32_t block, int x, int y, uint32_t lane) const {
        const uint32_t unit = lane & 7u;
        const int col = x + int(unit) * 4;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t row = i * 4u + (lane >> 3);
            const float4 v = ptx::ld_shared_v4(block + row * 128u + ((unit ^ (row & 7u)) << 4));
            const int gr = y + int(row);
            if (gr < this->m && col < this->n)
                ptx::multimem_st_v4(mc_c + static_cast<long long>(gr) * this->ldc + col, v);
        }
    }
    // Two staged blocks side by side (columns [x, x + 64)): each instruction of the warp covers two
    // rows of 256 contiguous bytes, the largest payload an NVLink write carries.
    __device__ __forceinline__ void multimem_store_pair(uint32_t block, int x, int y, uint32_t lane) const {
        const uint32_t u = lane & 15u, blk = u >> 3, unit = u & 7u;
        const int col = x + int(u) * 4;
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i) {
            const uint32_t row = i * 2u + (lane >> 4);
            const float4 v = ptx::ld_shared_v4(block + blk * 4096u + row * 128u + ((unit ^ (row & 7u)) << 4));
            const int gr = y + int(row);
            if (gr < this->m && col < this->n)
                ptx::multimem_st_v4(mc_c + static_cast<long long>(gr) * this->ldc + col, v);
        }
    }
};

// Zeroes the C region of tiles [first_tile, first_tile + gridDim.x) (raster order); blockIdx.y
// selects a band of 16 rows inside the tile.
__global__ void zero_tiles_kernel(float* __restrict__ c, long long ldc, int m, int n, int tile_m, int tile_n,
                                  int tiles_m, int tiles_n, int raster_group, int first_tile, int vec_ok) {
    int tm, tn;
    raster_coords(first_tile + blockIdx.x, tiles_m, tiles_n, raster_group, tm, tn);
    const int row0 = tm * tile_m + blockIdx.y * 16, col0 = tn * tile_n;
    const int rows = min(16, m - row0), cols = min(tile_n, n - col0);
    if (rows <= 0 || cols <= 0) return;
    if (vec_ok && cols % 4 == 0) {
        const int vcols = cols / 4;
        for (int i = threadIdx.x; i < rows * vcols; i += blockDim.x) {
            const int r = i / vcols, q = i - r * vcols;
            *reinterpret_cast<float4*>(c + static_cast<long long>(row0 + r) * ldc + col0 + q * 4) =
                make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    } else {
        for (int i = threadIdx.x; i < rows * cols; i += blockDim.x) {
            const int r = i / cols, q = i - r * cols;
            c[static_cast<long long>(row0 + r) * ldc + col0 + q] = 0.0f;
        }
    }
}

// Whether a CTA's last tile stages its results in the idle stage ring (see umma_gemm.cuh).
constexpr bool kRingStagingDefault = true;

// OUT: 0 = C on this GPU; 1 = also stored into the peers' C (bulk tensor stores); 2 = stored through a
// multicast address into every GPU's C.
template <int CTAS, int BN, bool B_MN_MAJOR, int KATOMS, bool A_MN_MAJOR = false, int OUT = 0>
void launch_variant(const float* a, const float* b, float* c, int m, int n, int k,
                    const UmmaEpilogueArgs& epi, const GemmTuning& tune, cudaStream_t stream,
                    const GemmPeerOutputs* peers = nullptr, float* mc_c = nullptr) {
    using Cfg = UmmaConfig<CTAS, BN, B_MN_MAJOR, KATOMS>;
    constexpr bool PUSH = OUT == 1;
    using Prob = std::conditional_t<OUT == 1, GemmPushProblem<CTAS, BN, B_MN_MAJOR>,
                                    std::conditional_t<OUT == 2, GemmMultimemProblem<CTAS, BN, B_MN_MAJOR>,
                                                       GemmProblem<CTAS, BN, B_MN_MAJOR, A_MN_MAJOR>>>;
    static_assert(!(OUT != 0 && A_MN_MAJOR), "peer stores are built for the forward layouts only");
    const DeviceInfo& dev = device_info();

    Prob prob;
    prob.a_chunked = 0;
    if (A_MN_MAJOR && m % 32 == 0) {
        // A stored [K, M]: M/32 column chunks of 32 floats, one box {32, 32, 4} per stage.
        const uint64_t dims[3] = {32, uint64_t(k), uint64_t(m / 32)};
        const uint64_t strides[2] = {uint64_t(m) * 4, 128};
        const uint32_t box[3] = {32, UMMA_BK, uint32_t(UMMA_BM / 32)};
        encode_tensor_map(&prob.map_a, a, 3, dims, strides, box, TmaSwizzle::B128Atom32);
        prob.a_chunked = 1;
    } else if (A_MN_MAJOR) {
        const uint64_t dims[2] = {uint64_t(m), uint64_t(k)};
        const uint64_t strides[1] = {uint64_t(m) * 4};
        const uint32_t box[2] = {32, UMMA_BK};
        encode_tensor_map(&prob.map_a, a, 2, dims, strides, box, TmaSwizzle::B128Atom32);
    } else {
        const uint64_t dims[2] = {uint64_t(k), uint64_t(m)};
        const uint64_t strides[1] = {uint64_t(k) * 4};
        const uint32_t box[2] = {UMMA_BK, UMMA_BM};
        encode_tensor_map(&prob.map_a, a, 2, dims, strides, box, TmaSwizzle::B128);
    }
    prob.b_chunked = 0;
    if (B_MN_MAJOR && n % 32 == 0 && tune.b_chunked >= 0) {
        // B[K,N] seen as N/32 column chunks of 32 floats: {32, K, N/32} with strides
        // {row pitch, 128 B}.  One box {32, 32, chunks} fills the stage in the order the
        // MMA descriptors expect (chunk-major, 4096 B per chunk).
        const uint64_t dims[3] = {32, uint64_t(k), uint64_t(n / 32)};
        const uint64_t strides[2] = {uint64_t(n) * 4, 128};
        const uint32_t box[3] = {32, UMMA_BK, uint32_t(Cfg::BN_CTA / 32)};
        encode_tensor_map(&prob.map_b, b, 3, dims, strides, box, TmaSwizzle::B128Atom32);
        prob.b_chunked = 1;
    } else if (B_MN_MAJOR) {
        const uint64_t dims[2] = {uint64_t(n), uint64_t(k)};
        const uint64_t strides[1] = {uint64_t(n) * 4};
        const uint32_t box[2] = {32, UMMA_BK};
        encode_tensor_map(&prob.map_b, b, 2, dims, strides, box, TmaSwizzle::B128Atom32);
    } else {
        const uint64_t dims[2] = {uint64_t(k), uint64_t(n)};
        const uint64_t strides[1] = {uint64_t(k) * 4};
        const uint32_t box[2] = {UMMA_BK, uint32_t(Cfg::BN_CTA)};
        encode_tensor_map(&prob.map_b, b, 2, dims, strides, box, TmaSwizzle::B128);
    }
    const bool tma_store = prob.set_output(c, m, n, tune.tma_store >= 0);
    if constexpr (PUSH) {
        CB200_REQUIRE(peers != nullptr && peers->count >= 0 && peers->count <= kMaxGemmPeers, "bad peer output list");
        CB200_REQUIRE(tma_store, "peer stores need bulk tensor stores: N % 4 == 0 and a 16-byte aligned C");
        prob.n_peers = peers->count;
        for (int i = 0; i < peers->count; ++i) {
            CB200_REQUIRE(peers->c[i] != nullptr && (reinterpret_cast<uintptr_t>(peers->c[i]) & 15u) == 0,
                          "peer C pointers must be 16-byte aligned");
            // The same view as map_c (this rank's rows only, so tiles that hang over the shard's
            // last row are clipped in every copy).
            const uint64_t dims[2] = {uint64_t(n), uint64_t(m)};
            const uint64_t strides[1] = {uint64_t(n) * 4};
            const uint32_t box[2] = {32, 32};
            encode_tensor_map(&prob.peer_c[i], peers->c[i], 2, dims, strides, box, TmaSwizzle::B128);
        }
    }

    UmmaSchedule sched = whole_tile_schedule(
        (m + UMMA_BM * CTAS - 1) / (UMMA_BM * CTAS), (n + BN - 1) / BN, (k + UMMA_BK - 1) / UMMA_BK, BN,
        Cfg::TX_BYTES, (tune.stages > 0 && tune.stages < Cfg::STAGES) ? tune.stages : Cfg::STAGES, dev.status_word);
    if (tune.raster_group > 0) sched.raster_group = tune.raster_group;
    sched.b_lbo = tune.b_lbo;
    sched.b_sbo = tune.b_sbo;
    sched.tma_store = tma_store ? 1 : 0;
    sched.debug = tune.debug;
    if (tune.wait_limit_ms > 0) sched.wait_limit_ns = static_cast<unsigned long long>(tune.wait_limit_ms) * 1000000ull;
    const uint32_t whole_tile_staging = tma_store ? UMMA_STORE_STAGING_BYTES : 0u;

    const int num_tiles = sched.tiles_m * sched.tiles_n;
    int max_ctas = tune.max_ctas > 0 ? tune.max_ctas : dev.num_sms;
    int groups = max_ctas / CTAS;
    if (groups < 1) groups = 1;

    // Split-K: when the last wave of tiles leaves most of the machine idle, cut each of its
    // tiles into K ranges so that the wave is both full and proportionally shorter.
    sched.n_whole = num_tiles;
    sched.split = 1;
    sched.kb_per_split = sched.k_blocks;
    const int tail = num_tiles % groups;
    int want_split = tune.split_k;
    if (want_split == 0 && epi.act == EPI_NONE && tail > 0 && num_tiles > groups && sched.k_blocks >= 16) {
        // Only behind at least one full wave (for a problem that does not fill the machine the
        // zeroing pass and the atomic adds cost more than the shorter K loop saves), and two
        // ranges at most when choosing automatically: their sum does not depend on the order in
        // which they arrive, so results stay bitwise reproducible.
        want_split = groups / tail >= 2 ? 2 : 1;
    }
    if (want_split >= 2 && epi.act == EPI_NONE && tail > 0) {
        int per = (sched.k_blocks + want_split - 1) / want_split;
        per = (per + KATOMS - 1) / KATOMS * KATOMS;
        const int parts = (sched.k_blocks + per - 1) / per;
        if (parts >= 2) {
            sched.n_whole = num_tiles - tail;
            sched.split = parts;
            sched.kb_per_split = per;
            zero_tiles_kernel<<<dim3(tail, UMMA_BM * CTAS / 16), 256, 0, stream>>>(
                c, prob.ldc, m, n, UMMA_BM * CTAS, BN, sched.tiles_m, sched.tiles_n, sched.raster_group,
                sched.n_whole, prob.vec_ok);
            CB200_CHECK_LAUNCH();
        }
    }
    const int num_units = sched.n_whole + (num_tiles - sched.n_whole) * sched.split;
    if (groups > num_units) groups = num_units;

    // Split-K inside a cluster, for problems with far fewer tiles than SMs: one cluster of
    // CTAS * ksplit CTAs per tile, partial sums exchanged through distributed shared memory.
    int ksplit = (sched.split == 1) ? tune.cluster_split : 1;
    int per = sched.k_blocks;
    uint32_t exchange_bytes = 0;
    while (ksplit > 1) {
        per = (sched.k_blocks + ksplit - 1) / ksplit;
        per = (per + KATOMS - 1) / KATOMS * KATOMS;
        exchange_bytes = uint32_t(ksplit - 1) * UMMA_BM * (BN / ksplit) * 4u;
        // (A split tile stages its stores in the idle stage ring: no staging area of its own.)
        const bool fits = exchange_bytes + 2 * Cfg::STAGE_BYTES <= Cfg::SMEM_BUDGET;
        if (CTAS * ksplit <= 8 && BN % (32 * ksplit) == 0 && (sched.k_blocks + per - 1) / per == ksplit && fits)
            break;
        ksplit /= 2;
    }
    sched.cluster_split = 1;
    if (ksplit > 1) {
        sched.cluster_split = ksplit;
        sched.kb_per_split = per;
        groups = num_tiles * ksplit;
    } else {
        exchange_bytes = 0;
    }
    sched.exchange_bytes = exchange_bytes;
    // Dynamic shared memory: [stages][exchange buffer][store staging], after up to 1 KB of alignment.
    const uint32_t staging_bytes = ksplit > 1 ? 0u : whole_tile_staging;
    const int fit_stages = int((Cfg::SMEM_BUDGET - exchange_bytes - staging_bytes) / Cfg::STAGE_BYTES);
    if (sched.stages > fit_stages) sched.stages = fit_stages;
    const bool ring_wanted = kRingStagingDefault != (tune.ring_staging < 0);      // the tuning flag flips the default
    sched.ring_staging = (uint32_t(sched.stages) * Cfg::STAGE_BYTES >= 131072u && ring_wanted) ? 1 : 0;
    const uint32_t smem_bytes = uint32_t(sched.stages) * Cfg::STAGE_BYTES + exchange_bytes + staging_bytes + 1024;

    if constexpr (OUT == 2) {
        CB200_REQUIRE(tma_store && mc_c != nullptr && (reinterpret_cast<uintptr_t>(mc_c) & 15u) == 0,
                      "multicast stores need N % 4 == 0 and a 16-byte aligned multicast address of C");
        prob.mc_c = mc_c;
    }
    if constexpr (OUT != 0)
        CB200_REQUIRE(sched.split == 1 && sched.cluster_split == 1 && sched.tma_store == 1,
                      "peer stores need whole tiles written through the staging blocks");
    CB200_TRACE("gemm tf32 tcgen05: M=%d N=%d K=%d A=%s B=%s tile=%dx%d ctas/mma=%d katoms=%d stages=%d "
                "clusters=%d x %d CTAs tail_split=%d cluster_split=%d store=%s peers=%d act=%d bias=%d",
                m, n, k, A_MN_MAJOR ? "[K,M]" : "[M,K]", B_MN_MAJOR ? "[K,N]" : "[N,K]", UMMA_BM * CTAS, BN, CTAS,
                KATOMS, sched.stages, groups / sched.cluster_split, CTAS * sched.cluster_split, sched.split,
                sched.cluster_split, sched.tma_store ? "bulk-tensor" : "registers",
                PUSH ? (peers ? peers->count : 0) : 0, epi.act, epi.bias != nullptr);
    auto kernel = umma_tf32_kernel<CTAS, BN, B_MN_MAJOR, KATOMS, Prob, A_MN_MAJOR>;
    // `groups` counts CTA groups (a CTA or a pair); a cluster holds cluster_split of them.
    launch_umma(kernel, prob, sched, epi, groups / sched.cluster_split, CTAS * sched.cluster_split, smem_bytes,
                Cfg::SMEM_MAX, stream);
}

// One tile shape with what it costs, measured on B200 at 1.9 GHz with cold operands (launches
// back to back in a CUDA graph):
//   step_ns   one K = 8 step of a CTA in the steady state.  The MMA reads both operands from
//             shared memory at about 96 B/clk and an SM takes in about 60 B/clk from L2, so narrow
//             tiles pay per step for bytes, not for flops; a CTA pair halves the B bytes per CTA.
//   base_us   launch, set-up, first loads and teardown (clusters cost more);
//   epi_us    reading one accumulator out of TMEM and storing the CTA's part of the tile.
struct TileCost { int ctas, bn; double step_ns, base_us, epi_us; };
constexpr TileCost kTileCosts[] = {
    {2, 256, 80.0, 4.9, 4.0}, {1, 256, 97.0, 3.9, 4.0}, {2, 128, 53.0, 4.9, 2.5},
    {1, 128, 68.0, 3.9, 2.5}, {1, 64, 54.0, 3.9, 1.7}};

struct TilePick { int ctas, bn, cluster_split, katoms; };

// Pipeline stages left for a configuration once the exchange buffer and the store staging are
// taken from the CTA's shared memory.
inline int stages_for(int ctas, int bn, int katoms, int cluster_split) {
    const int stage = katoms * (int(UMMA_BM) * UMMA_BK * 4 + bn / ctas * UMMA_BK * 4);
    const int exchange = cluster_split > 1 ? (cluster_split - 1) * UMMA_BM * (bn / cluster_split) * 4 : 0;
    const int staging = cluster_split > 1 ? 0 : int(UMMA_STORE_STAGING_BYTES);      // split tiles stage in the ring
    const int budget = 232448 - 1024 - 512 - exchange - staging;
    const int stages = budget / stage;
    return stages > 8 ? 8 : stages;
}

inline int default_katoms(int ctas, int bn, int cluster_split) {
    // Two K blocks per stage halve the barrier traffic of the MMA issuer; taken wherever at
    // least three such stages fit.
    if (ctas == 1 && bn == 256) return 1;
    return stages_for(ctas, bn, 2, cluster_split) >= 3 ? 2 : 1;
}

// Estimated time of one configuration in microseconds (0 when it cannot run).
inline double estimate_us(const TileCost& t, int cluster_split, int m, int n, int k, bool allow_tail_split,
                          int num_sms) {
    const long long tiles = static_cast<long long>((m + 128 * t.ctas - 1) / (128 * t.ctas)) * ((n + t.bn - 1) / t.bn);
    const int k_blocks = (k + UMMA_BK - 1) / UMMA_BK;
    // Operands cross HBM at least once.
    const double dram_us = (double(m) * k + double(n) * k + double(m) * n) * 4.0 / 6.5e6;
    if (cluster_split == 1) {
        const long long slots = num_sms / t.ctas;
        const long long tail = tiles % slots;
        double waves = double(tiles / slots) + (tail > 0 ? 1.0 : 0.0);
        double extra = 0.0;
        if (allow_tail_split && tail > 0 && tiles > slots && slots / tail >= 2 && k_blocks >= 16) {
            waves -= 0.5;            // the ragged last wave is cut in two K ranges
            extra = 1.5;             // zeroing C, adding partial sums
        }
        const double loop_us = waves * 4.0 * k_blocks * t.step_ns * 1e-3;
        return t.base_us + (loop_us > dram_us ? loop_us : dram_us) + t.epi_us + extra;
    }
    // Split-K inside a cluster: one cluster of ctas * cluster_split CTAs per tile.  Clusters of
    // more than two CTAs live inside one GPC and do not pack the SMs completely.
    const int cluster = cluster_split * t.ctas;
    const long long cluster_slots = cluster <= 2 ? num_sms / cluster : static_cast<long long>(num_sms * 0.875 / cluster + 0.5);
    const int per = (k_blocks + cluster_split - 1) / cluster_split;
    if (cluster > 8 || tiles > cluster_slots || t.bn % (32 * cluster_split) != 0 || per < 2 ||
        (k_blocks + per - 1) / per != cluster_split)
        return 0.0;
    const int katoms = default_katoms(t.ctas, t.bn, cluster_split);
    if (stages_for(t.ctas, t.bn, katoms, cluster_split) < 2) return 0.0;
    // The exchange: a fixed part, the 32-column chunks a CTA sends (and as many it adds up), and
    // what wider clusters cost beyond that (fitted to graph-timed launches from 512^3 to
    // 128 x 4096 x 4096 after the exchange became asynchronous stores).
    double exchange_us = 1.0 + 0.45 * (t.bn / 32) * (cluster_split - 1) / cluster_split;
    for (int s = cluster_split; s > 2; s /= 2) exchange_us += 0.75;
    const double loop_us = 4.0 * per * t.step_ns * 1e-3;
    return t.base_us + (loop_us > dram_us ? loop_us : dram_us) + t.epi_us / cluster_split + exchange_us;
}

template <bool A_MN_MAJOR>
TilePick pick_tile(int m, int n, int k, const UmmaEpilogueArgs& epi, const GemmTuning& tune, int num_sms) {
    TilePick pick{1, 64, 1, 0};
    double best = 0.0;
    for (const TileCost& t : kTileCosts) {
        if (tune.ctas != 0 && t.ctas != tune.ctas) continue;
        if (tune.bn != 0 && t.bn != tune.bn) continue;
        if (A_MN_MAJOR && t.bn != 256) continue;          // the transposed-A kernels are built 256 wide only
        for (int ks = 1; ks <= 8; ks *= 2) {
            if (ks > 1 && (A_MN_MAJOR || tune.cluster_split == 1)) break;
            // 256-wide tiles keep too few pipeline stages beside their exchange buffer to gain
            // from a split (measured), so only narrower ones are split unless the caller insists.
            if (ks > 1 && t.bn == 256 && tune.cluster_split == 0) break;
            if (tune.cluster_split > 1 && ks != tune.cluster_split) continue;
            const bool tail_split = epi.act == EPI_NONE && tune.split_k != 1;
            const double us = estimate_us(t, ks, m, n, k, tail_split, num_sms);
            if (us > 0.0 && (best == 0.0 || us < best)) {
                best = us;
                pick = TilePick{t.ctas, t.bn, ks, 0};
            }
        }
    }
    return pick;
}

template <bool B_MN_MAJOR, bool A_MN_MAJOR = false>
void dispatch(const float* a, const float* b, float* c, int m, int n, int k,
              const UmmaEpilogueArgs& epi, const GemmTuning& tune, cudaStream_t stream) {
    const DeviceInfo& dev = device_info();
    int ctas = tune.ctas;
    int bn = tune.bn;
    int cluster_split = tune.cluster_split > 1 ? tune.cluster_split : 1;
    if (ctas == 0 || bn == 0) {
        const TilePick pick = pick_tile<A_MN_MAJOR>(m, n, k, epi, tune, dev.num_sms);
        ctas = pick.ctas;
        bn = pick.bn;
        cluster_split = pick.cluster_split;
    }
    int katoms = tune.katoms;
    if (katoms == 0) katoms = default_katoms(ctas, bn, cluster_split);
    GemmTuning chosen = tune;
    chosen.cluster_split = cluster_split;
#define CB200_CASE(C, N, KA)                                                              \
    if (ctas == C && bn == N && katoms == KA) {                                           \
        launch_variant<C, N, B_MN_MAJOR, KA, A_MN_MAJOR>(a, b, c, m, n, k, epi, chosen, stream); \
        return;                                                                           \
    }
    CB200_CASE(1, 256, 1)
    CB200_CASE(2, 256, 1)
    CB200_CASE(2, 256, 2)
    if constexpr (!A_MN_MAJOR) {      // narrow tiles are built for the forward layouts only
        CB200_CASE(1, 128, 1)
        CB200_CASE(1, 128, 2)
        CB200_CASE(1, 64, 1)
        CB200_CASE(1, 64, 2)
        CB200_CASE(2, 128, 1)
        CB200_CASE(2, 128, 2)
    }
#undef CB200_CASE
    CB200_REQUIRE(false, "unsupported TF32 GEMM tile configuration");
}

}  // namespace

GemmPlan gemm_tf32_plan(int m, int n, int k, int act, int num_sms) {
    CB200_REQUIRE(m > 0 && n > 0 && k > 0 && num_sms > 0, "gemm plan: extents and SM count must be positive");
    const UmmaEpilogueArgs epi{nullptr, 0, act};
    const GemmTuning tune;
    const TilePick pick = pick_tile<false>(m, n, k, epi, tune, num_sms);
    GemmPlan plan{pick.ctas, pick.bn, pick.cluster_split, default_katoms(pick.ctas, pick.bn, pick.cluster_split), 0.0};
    for (const TileCost& t : kTileCosts)
        if (t.ctas == pick.ctas && t.bn == pick.bn)
            plan.estimate_us = estimate_us(t, pick.cluster_split, m, n, k, act == EPI_NONE, num_sms);
    return plan;
}

bool gemm_tf32_supported(const float* a, const float* b, const float* c, int m, int n, int k,
                         bool b_is_nk) {
    if (m < 1 || n < 1 || k < 1) return false;
    if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u)) return false;
    (void)c;
    if (k % 4 != 0) return false;               // A rows (and W rows) must be 16-byte multiples
    if (!b_is_nk && n % 4 != 0) return false;   // B[K,N] rows likewise
    return device_info().cc_major == 10;
}

bool gemm_tf32_tn_supported(const float* a, const float* b, int m, int n, int k) {
    if (m < 1 || n < 1 || k < 1) return false;
    if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u)) return false;
    if (m % 4 != 0 || n % 4 != 0) return false;      // rows of A[K,M] and B[K,N] must be 16-byte multiples
    return device_info().cc_major == 10;
}

void gemm_tf32_tn(const float* a, const float* b, float* c, int m, int n, int k, const GemmTuning& tune,
                  cudaStream_t stream) {
    CB200_REQUIRE(gemm_tf32_tn_supported(a, b, m, n, k),
                  "TF32 tensor-core GEMM (transposed A) needs an sm_100 device, 16-byte aligned operands "
                  "and M, N multiples of 4");
    UmmaEpilogueArgs epi{nullptr, 0, EPI_NONE};
    GemmTuning t = tune;
    if (t.ctas == 0) t.ctas = (static_cast<long long>((m + 255) / 256) * ((n + 255) / 256) * 2 >= device_info().num_sms) ? 2 : 1;
    if (t.bn == 0) t.bn = 256;                        // only the 256-wide tiles are built for this layout
    CB200_REQUIRE(t.bn == 256, "transposed-A GEMM supports 256-wide tiles only");
    dispatch<true, true>(a, b, c, m, n, k, epi, t, stream);
}

void gemm_tf32_push(const float* a, const float* b, bool b_is_nk, float* c, int m, int n, int k,
                    const GemmPeerOutputs& peers, const GemmTuning& tune, cudaStream_t stream) {
    CB200_REQUIRE(gemm_tf32_supported(a, b, c, m, n, k, b_is_nk) && n % 4 == 0,
                  "TF32 tensor-core GEMM with peer stores needs an sm_100 device, 16-byte aligned operands and "
                  "row lengths that are multiples of 4");
    UmmaEpilogueArgs epi{nullptr, 0, EPI_NONE};
    GemmTuning t = tune;
    t.split_k = 1;            // whole tiles only
    t.cluster_split = 1;
    t.tma_store = 0;
    // One tile shape: the CTA pair with a 256 x 256 tile (shards are large, that is what they take anyway).
    if (b_is_nk) launch_variant<2, 256, false, 2, false, 1>(a, b, c, m, n, k, epi, t, stream, &peers);
    else launch_variant<2, 256, true, 2, false, 1>(a, b, c, m, n, k, epi, t, stream, &peers);
}

void gemm_tf32_multimem(const float* a, const float* b, bool b_is_nk, float* c_local, float* c_multicast, int m, int n,
                        int k, const GemmTuning& tune, cudaStream_t stream) {
    CB200_REQUIRE(gemm_tf32_supported(a, b, c_local, m, n, k, b_is_nk) && n % 4 == 0,
                  "TF32 tensor-core GEMM with multicast stores needs an sm_100 device, 16-byte aligned operands "
                  "and row lengths that are multiples of 4");
    UmmaEpilogueArgs epi{nullptr, 0, EPI_NONE};
    GemmTuning t = tune;
    t.split_k = 1;
    t.cluster_split = 1;
    t.tma_store = 0;
    if (b_is_nk) launch_variant<2, 256, false, 2, false, 2>(a, b, c_local, m, n, k, epi, t, stream, nullptr, c_multicast);
    else launch_variant<2, 256, true, 2, false, 2>(a, b, c_local, m, n, k, epi, t, stream, nullptr, c_multicast);
}

void gemm_tf32(const float* a, const float* b, bool b_is_nk, float* c, int m, int n, int k,
               const float* bias, bool bias_per_row, int act, const GemmTuning& tune,
               cudaStream_t stream) {
    CB200_REQUIRE(gemm_tf32_supported(a, b, c, m, n, k, b_is_nk),
                  "TF32 tensor-core GEMM needs an sm_100 device, 16-byte aligned operands and "
                  "row lengths that are multiples of 4");
    UmmaEpilogueArgs epi{bias, bias_per_row ? 1 : 0, act};
    if (b_is_nk) dispatch<false>(a, b, c, m, n, k, epi, tune, stream);
    else dispatch<true>(a, b, c, m, n, k, epi, tune, stream);
}

}  // namespace cudeep_b200
