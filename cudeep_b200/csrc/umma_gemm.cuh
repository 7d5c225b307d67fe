// Persistent, warp-specialised TF32 GEMM mainloop for sm_100a.
//
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor loads)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma; the warp owns TMEM)
//   warps 2..5  epilogue       (tcgen05.ld -> bias/activation -> 128-bit stores)
//
// A CTA owns 128 accumulator rows.  With CTAS == 2 two CTAs of a cluster form a
// pair: the tile is 256 x BN, each CTA stages its own 128 rows of A and its own
// half of B, and the pair's leader (cluster rank 0) issues cta_group::2 MMAs
// that read both CTAs' shared memory.  No load is multicast.
//
// The accumulator lives in TMEM and is double-buffered (2 x BN columns) so the
// epilogue of tile i overlaps the mainloop of tile i+1.
//
// The kernel is shared by the dense GEMM / Linear forward and the
// implicit-GEMM convolution through a `Problem` policy that supplies the tile
// decode, the TMA loads of one K block and the output store.
#pragma once

#include "runtime.h"
#include "sm100_ptx.cuh"
#include "epilogue_math.cuh"

namespace cudeep_b200 {

// Codes written to the device status word when a bounded wait runs out.
enum UmmaStatus : uint32_t {
    UMMA_OK = 0,
    UMMA_TIMEOUT_PRODUCER = 1,   // producer waited for a free stage
    UMMA_TIMEOUT_MMA_FULL = 2,   // MMA issuer waited for operand data
    UMMA_TIMEOUT_MMA_ACC = 3,    // MMA issuer waited for a free accumulator
    UMMA_TIMEOUT_EPILOGUE = 4,   // epilogue waited for a finished accumulator
    UMMA_TIMEOUT_EXCHANGE = 5,   // epilogue waited for the partial sums of the other K ranges
};

constexpr int UMMA_BM = 128;        // accumulator rows per CTA
constexpr int UMMA_BK = 32;         // fp32 elements per K block = one 128-byte swizzle row
constexpr int UMMA_K = 8;           // K of one tcgen05.mma kind::tf32
constexpr int UMMA_THREADS = 192;

struct UmmaEpilogueArgs {
    const float* bias;     // nullptr = none
    int bias_per_row;      // 0: bias[column], 1: bias[row]
    int act;               // cudeep_b200 epilogue code (0 none, 1 relu, 2 gelu, 3 silu, 4 sigmoid)
};

struct UmmaSchedule {
    int tiles_m;           // tile rows  (tile = 128*CTAS rows)
    int tiles_n;           // tile columns
    int k_blocks;          // ceil(K / 32)
    int raster_group;      // tile rows walked together so concurrent CTAs share B columns in L2
    uint32_t* status;      // device status word
    unsigned long long wait_limit_ns;
    uint32_t b_lbo, b_sbo; // non-zero: override the B descriptor offsets (bring-up aid)
    int umma_n;            // N of one MMA (<= BN, multiple of 32): accumulator columns in use
    uint32_t tx_bytes;     // bytes all CTAs of the group deliver per stage (all atoms)
    int stages;            // pipeline stages in use (<= UmmaConfig::STAGES)
    // Split-K for the ragged last wave (or for problems too small to fill the machine): the
    // first n_whole tiles (in raster order) are computed whole; each remaining tile is cut
    // into `split` K ranges of kb_per_split blocks (a multiple of KATOMS), one work unit
    // each, whose partial sums are added into a zeroed C.  split == 1: every tile is whole.
    int n_whole;
    int split;
    int kb_per_split;
    // Split-K inside a thread-block cluster (cluster_split > 1; then split == 1): a cluster of
    // CTAS * cluster_split CTAs owns one tile, CTA group g of it accumulates K blocks
    // [g * kb_per_split, (g + 1) * kb_per_split), and the groups exchange partial sums through
    // distributed shared memory: group g receives columns [g, g + 1) * umma_n / cluster_split of
    // every other group's accumulator, adds them to its own in a fixed order and stores that
    // slice with bias and activation.  The grid holds one cluster per tile, the exchange buffer
    // starts `stages` stages into the dynamic shared memory, and every group has a non-empty
    // K range.
    int cluster_split;
    uint32_t exchange_bytes;   // size of that exchange buffer (0 without cluster split)
    // Problems with a tensor map of the output (Problem::kTmaStore, and the launch says so here)
    // stage each 32 x 32 block of results in shared memory, behind the stages and the exchange
    // buffer, and write it with one bulk tensor store: 8 KB (two blocks) per epilogue warp.
    int tma_store;
    int ring_staging;      // the stages in use span at least 128 KB: the last tile's epilogue may stage in them
    int plane_store;       // Problem::kPlaneStore and the launch qualifies: see has_plane_store
    // Diagnostics for performance bring-up (results are then meaningless):
    //   bit 0: after the ring has been filled once the producer stops loading and only
    //          signals the stages, so the MMA side runs without memory traffic;
    //   bit 1: the MMA issuer skips the MMAs and only recycles stages, so the load side
    //          runs alone;
    //   bit 2: the MMA issuer ignores the stage ring (no waits, no stage commits) and the
    //          producer does nothing: raw MMA issue rate;
    //   bit 3: the epilogue neither reads TMEM nor stores;
    //   bit 4: the bulk-store epilogue stages its results but issues no store;
    //   bit 5: the bulk-store epilogue skips the accumulator loads;
    //   bit 7: the producer issues nothing at all, so the MMA issuer's bounded wait for operands
    //          runs out: the kernel must then record its status code, unwind every role, free
    //          its TMEM and return (the way to test that path without a fault).
    uint32_t debug;
};

// KATOMS: 32-wide K blocks ("atoms") per pipeline stage.  A stage is KATOMS
// consecutive [A atom][B atom] pairs; barriers are exchanged once per stage, so
// a larger KATOMS spends fewer of the MMA issuer's cycles on handshakes.
// Tile index -> tile coordinates: groups of `raster_group` tile rows are walked column by
// column, so CTAs working on consecutive tiles share operand slabs in L2.
__host__ __device__ inline void raster_coords(int t, int tiles_m, int tiles_n, int raster_group, int& tm,
                                              int& tn) {
    const int group_tiles = raster_group * tiles_n;
    const int group = t / group_tiles;
    const int first_m = group * raster_group;
    const int rows = (tiles_m - first_m) < raster_group ? (tiles_m - first_m) : raster_group;
    const int in_group = t - group * group_tiles;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

// One unit of work of the persistent loop: a tile and a range of its K blocks.
struct WorkUnit {
    int tile;
    int kb0;        // first K block
    int kb_count;   // K blocks in this unit
    int mode;       // 0: whole tile, plain store; 1: first K range of a split tile; 2: a later range
};

template <int CTAS, int BN, bool B_MN_MAJOR, int KATOMS = 1>
struct UmmaConfig {
    static constexpr int BN_CTA = BN / CTAS;                       // B rows staged by one CTA
    static constexpr uint32_t A_BYTES = UMMA_BM * UMMA_BK * 4;     // one A atom
    static constexpr uint32_t B_BYTES = BN_CTA * UMMA_BK * 4;      // one B atom (at most)
    static constexpr uint32_t ATOM_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t STAGE_BYTES = ATOM_BYTES * KATOMS;
    static constexpr uint32_t TX_BYTES = STAGE_BYTES * CTAS;       // counted on the leader's barrier
    // 227 KB of shared memory per CTA, minus alignment slack and the barriers.
    static constexpr uint32_t SMEM_BUDGET = 232448 - 1024 - 512;
    static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES > 8 ? 8 : SMEM_BUDGET / STAGE_BYTES;
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + alignment slack
    static constexpr uint32_t SMEM_MAX = SMEM_BUDGET + 1024;              // most a launch may ask for
    static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;      // 128 / 256 / 512
    static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
    static_assert(CTAS == 1 || CTAS == 2, "CTAS must be 1 or 2");
};

// Problem policy contract:
//   struct Tile;                                             decoded tile coordinates
//   __device__ Tile decode(int tm, int tn, uint32_t cta_rank) const;
//   __device__ void load(tile, kb, a_smem, b_smem, bar) const;     one lane, issues all TMA loads of a stage
//   __device__ void store(tile, row_in_cta, col0, float (&v)[32], epi, mode) const;   32 consecutive
//       columns of one row; mode as WorkUnit::mode (1, 2: add the partial sum into C)
//   static constexpr bool kClusterSplit;   the launcher may set UmmaSchedule::cluster_split > 1
//   static constexpr bool kTmaStore;   if true, also:
//   __device__ void finish(tile, row_in_cta, col0, float (&v)[32], epi) const;   bias + activation only
//   __device__ const CUtensorMap* out_map() const;      C as {N, M}, box {32, 32}, 128-byte swizzle
//   __device__ void out_coords(tile, row_in_cta, col0, int& x, int& y) const;
constexpr uint32_t UMMA_STORE_STAGING_BYTES = 4 * 2 * 4096;     // 4 epilogue warps x 2 blocks of 32 x 32 floats
// KIND: 0 = FP32 operands multiplied as TF32 (K block of 32 elements), 1 = FP16 operands, 2 = BF16
// operands (K block of 64 elements); a K block is 128 bytes per operand row either way, so stages,
// barriers and the epilogue do not change.
constexpr int UMMA_KIND_TF32 = 0;
constexpr int UMMA_KIND_F16 = 1;
constexpr int UMMA_KIND_BF16 = 2;

// Optional part of the problem contract, for a row-sharded product whose every rank needs all of C:
//   static constexpr bool kPeerStore = true;
//   __device__ void push(uint32_t block, int x, int y) const;
// push() repeats the bulk tensor store of a staged 32 x 32 block into the copies of C that live in
// the other GPUs' memory (tensor maps over peer-mapped addresses): the all-gather of C rides on the
// epilogue, tile by tile, instead of following the GEMM as a collective.  Stores only - no load in
// this kernel ever names peer memory.
template <class P, class = void>
struct has_peer_store { static constexpr bool value = false; };
template <class P>
struct has_peer_store<P, decltype((void)P::kPeerStore)> { static constexpr bool value = P::kPeerStore; };

template <class P>
__device__ __forceinline__ void push_to_peers(const P& prob, uint32_t block, int x, int y) {
    if constexpr (has_peer_store<P>::value) prob.push(block, x, y);
}

// The other optional form of the same idea:
//   static constexpr bool kMultimemStore = true;
//   __device__ void multimem_store(uint32_t block, int x, int y, uint32_t lane) const;
//   __device__ void multimem_store_pair(uint32_t block, int x, int y, uint32_t lane) const;   two blocks, 64 columns
// The whole warp reads the staged 32 x 32 block back (4 rows of 128 bytes per instruction) and writes
// it with multimem.st through a multicast address of C: one store travels over NVLink once and the
// switch replicates it into every GPU's copy, this GPU's included, so no bulk tensor store is issued.
template <class P, class = void>
struct has_multimem_store { static constexpr bool value = false; };
template <class P>
struct has_multimem_store<P, decltype((void)P::kMultimemStore)> { static constexpr bool value = P::kMultimemStore; };

// A third optional form, for tiles whose columns are several whole small output planes (a
// convolution over 7 x 7 maps): the accumulator columns of one plane, with the padding columns of
// its pixel box dropped, form a run of contiguous floats per row, and 32 consecutive rows form one
// contiguous block of the output.  So a warp compacts its 32 rows of one plane into its staging
// block and writes them with a single untiled bulk copy.
//   static constexpr bool kPlaneStore = true;
//   __device__ int plane_columns() const;           accumulator columns per plane (a multiple of 32)
//   __device__ uint32_t plane_bytes() const;        bytes of 32 rows of one compacted plane (<= 8192)
//   __device__ void plane_stage(uint32_t staging, uint32_t lane, int col_in_plane, const float (&v)[32]) const;
//   __device__ float* plane_dst(tile, int row0, int plane) const;    nullptr: nothing to write
// UmmaSchedule::plane_store switches it on for a launch (the staging blocks must then exist).
template <class P, class = void>
struct has_plane_store { static constexpr bool value = false; };
template <class P>
struct has_plane_store<P, decltype((void)P::kPlaneStore)> { static constexpr bool value = P::kPlaneStore; };

// One more optional form, for a 3 x 3 (or other KW-wide) stride-1 convolution over whole output rows:
//   static constexpr bool kSharedB = true;
// A pipeline stage then holds KATOMS A atoms - the filter slabs of the KATOMS taps of one filter row -
// and ONE B block: the rows of input pixels under that filter row, halo columns included, loaded once.
// Tap j's B operand is the same block read from j rows (pixels) further on: its descriptor starts
// j * 128 bytes later and is otherwise unchanged, base-offset field included (measured: the tensor
// core derives the 128-byte swizzle from the address bits, as TMA does when it writes the rows, so a
// block can be read from any row on; a base offset of j gives wrong products).  The pixel gather, the costliest
// requests of the TMA unit, shrinks by the filter width.  The schedule's K blocks count stages, the
// problem loads a whole stage at once (`load_stage`), and tiles leave row by row (`kRowStore`):
//   __device__ void load_stage(tile, int stage_index, uint32_t stage_smem, uint32_t b_smem, uint32_t bar) const;
//   __device__ int out_rows() const;                     output rows per tile
//   __device__ uint32_t row_column(int r) const;         first accumulator column of output row r
//   __device__ int row_values() const;                   values per row (<= 64)
//   __device__ void row_coords(tile, int row0, int r, int& x, int& y, int& z) const;   for out_map()
//   finish() as for kTmaStore; out_map() is a 3-D map {OW, OH, planes}, box {OW, 1, 32}, no swizzle.
// The mirror image for a grad_weight (B = input pixels as the K rows of an MN-major operand, A =
// grad_output, shared by all taps): `static constexpr int kTapShift = T;` (and `kTapColumns`).
// A stage is one ordinary atom whose B box is T - 1 pixels longer than the K block; tap t multiplies
// the same A with the B rows from t on (start address t * 128 bytes later) into its own kTapColumns
// accumulator columns, so one load of the input pixels serves the T taps of a filter row.  The B
// descriptor's leading-dimension offset comes from the schedule (b_lbo: the box's rows x 128 bytes).
template <class P, class = void>
struct tap_shift_of { static constexpr int value = 0; };
template <class P>
struct tap_shift_of<P, decltype((void)P::kTapShift)> { static constexpr int value = P::kTapShift; };
template <class P, class = void>
struct tap_columns_of { static constexpr int value = 0; };
template <class P>
struct tap_columns_of<P, decltype((void)P::kTapColumns)> { static constexpr int value = P::kTapColumns; };

template <class P, class = void>
struct has_shared_b { static constexpr bool value = false; };
template <class P>
struct has_shared_b<P, decltype((void)P::kSharedB)> { static constexpr bool value = P::kSharedB; };

template <int CTAS, int BN, bool B_MN_MAJOR, int KATOMS, class Problem, bool A_MN_MAJOR = false,
          int KIND = UMMA_KIND_TF32>
__global__ void __launch_bounds__(UMMA_THREADS, 1)
umma_tf32_kernel(const __grid_constant__ Problem prob, const UmmaSchedule sched,
                 const UmmaEpilogueArgs epi) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM101_ALL) || \
    defined(__CUDA_ARCH_FEAT_SM103_ALL)
    using Cfg = UmmaConfig<CTAS, BN, B_MN_MAJOR, KATOMS>;
    constexpr bool SHARED_B = has_shared_b<Problem>::value;
    constexpr uint32_t STAGE_BYTES = SHARED_B ? KATOMS * Cfg::A_BYTES + Cfg::B_BYTES : Cfg::STAGE_BYTES;
    constexpr int STAGES = SHARED_B ? int(Cfg::SMEM_BUDGET / STAGE_BYTES) : Cfg::STAGES;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ __align__(8) uint64_t bar_exchange;
    __shared__ uint32_t tmem_base_holder;
    __shared__ uint32_t abort_flag;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    // K ranges per tile (>= 1); problems that never split compile the exchange away.
    const uint32_t ksplit = Problem::kClusterSplit ? uint32_t(sched.cluster_split) : 1u;
    const bool clustered = (CTAS == 2) || ksplit > 1;
    const uint32_t cluster_rank = clustered ? ptx::cluster_ctarank() : 0u;
    const uint32_t cta_rank = (CTAS == 2) ? (cluster_rank & 1u) : 0u;       // place in the CTA pair
    const uint32_t kgroup = cluster_rank / CTAS;                            // which K range
    const uint32_t leader_rank = cluster_rank - cta_rank;                   // cluster rank of the pair's leader
    const bool is_leader = (cta_rank == 0);
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;

    ptx::WaitCtx wctx{&abort_flag, sched.status, sched.wait_limit_ns};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        prob.prefetch_maps();
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(ptx::smem_u32(&bar_acc_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_acc_empty[a]), 4 * CTAS);
        }
        // The exchange of a split tile: the other K ranges' partial sums arrive as asynchronous
        // stores that count their bytes on this barrier, (ksplit - 1) slices of 128 rows.
        ptx::mbar_init(ptx::smem_u32(&bar_exchange), 1);
        ptx::fence_mbar_init();
        if (ksplit > 1)
            ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bar_exchange),
                                       (ksplit - 1) * uint32_t(sched.umma_n) / ksplit * (UMMA_BM * 4u));
    }
    if (warp == 1) {
        ptx::tmem_alloc<CTAS>(ptx::smem_u32(&tmem_base_holder), Cfg::TMEM_COLS);
        ptx::tmem_relinquish<CTAS>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (clustered) {             // the peers' barriers must exist before anything signals them
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    ptx::tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;
    // Everything above touched only this launch's parameters and on-chip state, so it may overlap
    // the tail of the previous kernel in the stream.  So may what follows, up to the first access
    // to global memory of each role: the producer works out its first tile before it waits for the
    // predecessors (just before its first load), the epilogue warps wait before they first read a
    // bias or write C, and the MMA issuer touches only shared and tensor memory.
    ptx::grid_launch_dependents();

    const int num_tiles = sched.tiles_m * sched.tiles_n;
    const int num_units = sched.n_whole + (num_tiles - sched.n_whole) * sched.split;
    const int unit_stride = gridDim.x / (CTAS * ksplit);
    const int first_unit = blockIdx.x / (CTAS * ksplit);

    auto tile_coords = [&](int t, int& tm, int& tn) {
        raster_coords(t, sched.tiles_m, sched.tiles_n, sched.raster_group, tm, tn);
    };
    auto decode_unit = [&](int u) {
        WorkUnit w;
        if (ksplit > 1) {
            w.tile = u;
            w.kb0 = int(kgroup) * sched.kb_per_split;
            w.kb_count = min(sched.kb_per_split, sched.k_blocks - w.kb0);
            w.mode = 0;
        } else if (u < sched.n_whole) {
            w.tile = u;
            w.kb0 = 0;
            w.kb_count = sched.k_blocks;
            w.mode = 0;
        } else {
            const int r = u - sched.n_whole;
            const int part = r % sched.split;
            w.tile = sched.n_whole + r / sched.split;
            w.kb0 = part * sched.kb_per_split;
            w.kb_count = min(sched.kb_per_split, sched.k_blocks - w.kb0);
            w.mode = part == 0 ? 1 : 2;
        }
        return w;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && !(sched.debug & (4u | 0x80u))) {
            uint32_t stage = 0, phase = 0, issued = 0;
            for (int u = first_unit; u < num_units; u += unit_stride) {
                const WorkUnit w = decode_unit(u);
                int tm, tn;
                tile_coords(w.tile, tm, tn);
                const auto tile = prob.decode(tm, tn, cta_rank);
                const int k_stages = SHARED_B ? w.kb_count : (w.kb_count + KATOMS - 1) / KATOMS;
                if (u == first_unit) ptx::grid_dependency_wait();
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&bar_empty[stage]), phase ^ 1u, wctx,
                                        UMMA_TIMEOUT_PRODUCER))
                        goto producer_done;
                    const uint32_t full_local = ptx::smem_u32(&bar_full[stage]);
                    if ((sched.debug & 1u) && issued >= uint32_t(sched.stages)) {
                        if (is_leader) ptx::mbar_arrive(full_local);
                    } else {
                        if (is_leader) ptx::mbar_arrive_expect_tx(full_local, sched.tx_bytes);
                        const uint32_t full_bar = (CTAS == 2) ? ptx::mapa(full_local, leader_rank) : full_local;
                        // Atoms past the end of K are loaded too; their coordinates are out
                        // of range, so they arrive as zeros and add nothing.  (A split unit
                        // that is not the last holds a whole number of stages, so it never
                        // reaches into its neighbour's K range.)
                        if constexpr (SHARED_B) {
                            const uint32_t stage_smem = smem_base + stage * STAGE_BYTES;
                            prob.template load_stage<CTAS>(tile, w.kb0 + ks, stage_smem,
                                                           stage_smem + KATOMS * Cfg::A_BYTES, full_bar);
                        } else {
#pragma unroll
                            for (int j = 0; j < KATOMS; ++j) {
                                const uint32_t a_smem = smem_base + stage * STAGE_BYTES + j * Cfg::ATOM_BYTES;
                                prob.template load<CTAS>(tile, w.kb0 + ks * KATOMS + j, a_smem,
                                                         a_smem + Cfg::A_BYTES, full_bar);
                            }
                        }
                    }
                    ++issued;
                    if (++stage == uint32_t(sched.stages)) { stage = 0; phase ^= 1u; }
                }
            }
        }
    producer_done:
        __syncwarp();
        if (CTAS == 2) ptx::cluster_arrive();      // see the teardown
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (is_leader) {
            // All 32 lanes walk the loops together (a converged warp keeps descriptors and
            // addresses in the uniform datapath the tensor-core instructions read from); one
            // elected lane issues the MMAs and commits.
            const uint32_t idesc =
                KIND != UMMA_KIND_TF32
                    ? ptx::idesc_f16(UMMA_BM * CTAS, sched.umma_n, A_MN_MAJOR ? 1 : 0, B_MN_MAJOR ? 1 : 0,
                                     KIND == UMMA_KIND_BF16 ? 1 : 0)
                    : ptx::idesc_tf32(UMMA_BM * CTAS, sched.umma_n, /*a_mn=*/A_MN_MAJOR ? 1 : 0,
                                      /*b_mn=*/B_MN_MAJOR ? 1 : 0);
            // K-major operand: rows are 128 B, 8-row swizzle atoms 1024 B apart.
            // An MN-major A (a transposed left operand, stored [K, M]) uses the same layout as
            // an MN-major B: 32-row chunks 4096 B apart, 4-row K groups 512 B apart.
            const uint64_t a_base = A_MN_MAJOR ? ptx::smem_desc(4096, 512, ptx::SMEM_LAYOUT_SW128_ATOM32)
                                               : ptx::smem_desc(16, 1024, ptx::SMEM_LAYOUT_SW128);
            constexpr uint32_t a_kstep = A_MN_MAJOR ? 1024u : UMMA_K * 4u;
            // MN-major B (32-bit elements): the only layout the tensor core accepts is
            // the 128-byte swizzle with 32-byte atoms, whose pattern repeats every 4
            // K rows.  Each TMA box is 32 columns x 32 K rows (4096 B): column chunks
            // are 4096 B apart (LBO), 4-row K groups 512 B apart (SBO), and one MMA
            // (K = 8) advances the start address by 8 rows = 1024 B.
            // MN-major 16-bit B: the plain 128-byte swizzle; TMA boxes of 64 columns x 64 K rows
            // (8192 B): column chunks 8192 B apart, 8-row K groups 1024 B apart, and one MMA
            // (K = 16) advances by 16 rows = 2048 B.
            constexpr bool b_mn16 = B_MN_MAJOR && KIND != UMMA_KIND_TF32;
            const uint32_t b_lbo = sched.b_lbo ? sched.b_lbo : (b_mn16 ? 8192u : B_MN_MAJOR ? 4096u : 16u);
            const uint32_t b_sbo = sched.b_sbo ? sched.b_sbo : (b_mn16 ? 1024u : B_MN_MAJOR ? 512u : 1024u);
            const uint64_t b_base = ptx::smem_desc(
                b_lbo, b_sbo, (B_MN_MAJOR && !b_mn16) ? ptx::SMEM_LAYOUT_SW128_ATOM32 : ptx::SMEM_LAYOUT_SW128);
            constexpr uint32_t b_kstep = b_mn16 ? 2048u : B_MN_MAJOR ? 1024u : UMMA_K * 4u;
            const uint64_t a_desc0 = ptx::smem_desc_at(a_base, smem_base);
            const uint64_t b_desc0 =
                ptx::smem_desc_at(b_base, smem_base + (SHARED_B ? KATOMS * Cfg::A_BYTES : Cfg::A_BYTES));

            uint32_t stage = 0, phase = 0;
            int it = 0;
            for (int u = first_unit; u < num_units; u += unit_stride, ++it) {
                const int kb_count = decode_unit(u).kb_count;
                const int k_stages = SHARED_B ? kb_count : (kb_count + KATOMS - 1) / KATOMS;
                const uint32_t acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u,
                                                            wctx, UMMA_TIMEOUT_MMA_ACC)))
                    goto mma_done;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const bool free_run = (sched.debug & 4u) != 0;
                // The issuing thread is the critical path: every instruction between two
                // MMAs shows up as an idle tensor pipe.  So the barrier of the NEXT stage
                // is probed before this stage's MMAs are issued, and only waited on if
                // that early look found it incomplete.
                bool ready = free_run ||
                             __all_sync(0xffffffffu, ptx::mbar_test(ptx::smem_u32(&bar_full[stage]), phase));
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!ready) {
                        if (!__all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&bar_full[stage]), phase, wctx,
                                                                    UMMA_TIMEOUT_MMA_FULL)))
                            goto mma_done;
                    }
                    uint32_t next_stage = stage + 1, next_phase = phase;
                    if (next_stage == uint32_t(sched.stages)) { next_stage = 0; next_phase ^= 1u; }
                    ready = free_run || __all_sync(0xffffffffu, ptx::mbar_test(ptx::smem_u32(&bar_full[next_stage]),
                                                                               next_phase));
                    const bool issuer = ptx::elect_one();
                    if (issuer && !(sched.debug & 2u)) {
                        // Descriptors differ only in the start-address field (address >> 4),
                        // so each one is the stage's first descriptor plus a constant.
                        const uint64_t a_stage = a_desc0 + ((stage * STAGE_BYTES) >> 4);
                        const uint64_t b_stage = b_desc0 + ((stage * STAGE_BYTES) >> 4);
                        constexpr int TAP_SHIFT = tap_shift_of<Problem>::value;
                        if constexpr (TAP_SHIFT > 0) {
                            constexpr int TAP_COLS = tap_columns_of<Problem>::value;
                            const uint32_t idesc_tap =
                                ptx::idesc_tf32(UMMA_BM * CTAS, TAP_COLS, A_MN_MAJOR ? 1 : 0, B_MN_MAJOR ? 1 : 0);
#pragma unroll
                            for (int t = 0; t < TAP_SHIFT; ++t) {
#pragma unroll
                                for (int kk = 0; kk < UMMA_BK / UMMA_K; ++kk)
                                    ptx::umma_tf32<CTAS>(d_tmem + t * TAP_COLS, a_stage + ((kk * a_kstep) >> 4),
                                                         b_stage + ((t * 128u + kk * b_kstep) >> 4), idesc_tap,
                                                         (ks | kk) != 0);
                            }
                        } else {
#pragma unroll
                        for (int j = 0; j < KATOMS; ++j) {
#pragma unroll
                            for (int kk = 0; kk < UMMA_BK / UMMA_K; ++kk) {
                                // Shared B: atom j's A slab, and the one B block read from row j on
                                // (the start address j * 128 bytes later, nothing else).
                                const uint64_t a_desc =
                                    a_stage + (((SHARED_B ? j * Cfg::A_BYTES : j * Cfg::ATOM_BYTES) + kk * a_kstep) >> 4);
                                const uint64_t b_desc =
                                    SHARED_B ? b_stage + ((j * 128u + kk * b_kstep) >> 4)
                                             : b_stage + ((j * Cfg::ATOM_BYTES + kk * b_kstep) >> 4);
                                if constexpr (KIND != UMMA_KIND_TF32)
                                    ptx::umma_f16<CTAS>(d_tmem, a_desc, b_desc, idesc, (ks | j | kk) != 0);
                                else
                                    ptx::umma_tf32<CTAS>(d_tmem, a_desc, b_desc, idesc, (ks | j | kk) != 0);
                            }
                        }
                        }      // !TAP_SHIFT
                    }
                    // Free the stage once these MMAs have read it (in both CTAs of a pair).
                    if (issuer && !free_run) {
                        const uint32_t empty_local = ptx::smem_u32(&bar_empty[stage]);
                        ptx::umma_commit<CTAS>(empty_local);
                        if constexpr (CTAS == 2) ptx::umma_commit<CTAS>(ptx::mapa(empty_local, leader_rank + 1));
                    }
                    __syncwarp();
                    stage = next_stage;
                    phase = next_phase;
                }
                if (ptx::elect_one()) {
                    const uint32_t accf_local = ptx::smem_u32(&bar_acc_full[acc]);
                    ptx::umma_commit<CTAS>(accf_local);
                    if constexpr (CTAS == 2) ptx::umma_commit<CTAS>(ptx::mapa(accf_local, leader_rank + 1));
                }
                __syncwarp();
            }
        }
    mma_done:
        __syncwarp();
        if (CTAS == 2) ptx::cluster_arrive();
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t quarter = warp & 3u;            // TMEM lanes [32*quarter, +32) belong to this warp
        const int row_in_cta = quarter * 32 + lane;
        int it = 0;
        bool ok = true;
        uint32_t store_count = 0;      // bulk tensor stores issued by this warp
        for (int u = first_unit; u < num_units && ok; u += unit_stride, ++it) {
            const WorkUnit w = decode_unit(u);
            int tm, tn;
            tile_coords(w.tile, tm, tn);
            const auto tile = prob.decode(tm, tn, cta_rank);
            const uint32_t acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            ok = ptx::mbar_wait(ptx::smem_u32(&bar_acc_full[acc]), acc_phase, wctx,
                                UMMA_TIMEOUT_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (it == 0) ptx::grid_dependency_wait();      // before the first bias read or store to C
            ptx::tc_fence_after();
            const uint32_t t_row = tmem_base + acc * BN + ((quarter * 32u) << 16);
            // Two register sets: the TMEM load of the next 32 columns is in flight while the
            // current 32 are converted and stored.
            const int n_cols = (sched.debug & 8u) ? 0 : sched.umma_n;
            uint32_t r0[32], r1[32];
            // Writes 32 finished columns of this thread's row: through the staging block and a
            // bulk tensor store where the problem has an output map, else straight from registers.
            bool use_tma = false;
            if constexpr (Problem::kTmaStore) use_tma = sched.tma_store != 0 && w.mode == 0;
            // A tile split over a cluster is its CTA's only tile: when its epilogue starts the stage
            // ring is idle (every load was consumed by an MMA that has completed), so the staging
            // blocks lie at its start and no shared memory is set aside for them.
            const uint32_t staging = ksplit > 1 ? smem_base + quarter * 8192u
                                                : smem_base + uint32_t(sched.stages) * STAGE_BYTES +
                                                      sched.exchange_bytes + quarter * 8192u;
            auto emit = [&](int c, const uint32_t (&r)[32]) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                if constexpr (Problem::kTmaStore) {
                    if (use_tma) {
                        prob.finish(tile, row_in_cta, c, v, epi);
                        // The block written two stores ago must have been read out.
                        if (lane == 0) ptx::bulk_wait_group_read<1>();
                        __syncwarp();
                        const uint32_t block = staging + (store_count & 1u) * 4096u;
                        ++store_count;
                        const uint32_t row_smem = block + lane * 128u;
#pragma unroll
                        for (uint32_t q = 0; q < 8; ++q)      // 128-byte swizzle: unit q of row r at q ^ (r & 7)
                            ptx::st_shared_v4(row_smem + ((q ^ (lane & 7u)) << 4), v[4 * q], v[4 * q + 1],
                                              v[4 * q + 2], v[4 * q + 3]);
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            int x, y;
                            prob.out_coords(tile, int(quarter) * 32, c, x, y);
                            ptx::tma_store_2d(prob.out_map(), block, x, y);
                            push_to_peers(prob, block, x, y);
                            ptx::bulk_commit_group();
                        }
                        return;
                    }
                }
                if constexpr (has_plane_store<Problem>::value) {
                    if (sched.plane_store != 0) {
                        prob.finish(tile, row_in_cta, c, v, epi);
                        const int per_plane = prob.plane_columns();
                        const int plane = c / per_plane;
                        const int in_plane = c - plane * per_plane;
                        if (in_plane == 0) {      // the copy of the previous plane must have read the block
                            if (lane == 0) ptx::bulk_wait_group_read<0>();
                            __syncwarp();
                        }
                        prob.plane_stage(staging, lane, in_plane, v);
                        if (in_plane + 32 == per_plane) {
                            ptx::fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                float* dst = prob.plane_dst(tile, int(quarter) * 32, plane);
                                if (dst != nullptr) ptx::bulk_store_1d(dst, staging, prob.plane_bytes());
                                ptx::bulk_commit_group();
                            }
                        }
                        return;
                    }
                }
                prob.store(tile, row_in_cta, c, v, epi, w.mode);
            };
            if constexpr (SHARED_B && !has_plane_store<Problem>::value) {
                // ---- the tile leaves one output row at a time: its values are a run of accumulator
                // columns (the halo columns between rows are dropped), staged as a dense
                // [32 channels][values] block and written by one 3-D bulk tensor store.
                if constexpr (Problem::kTmaStore) {
                    const int out_rows = prob.out_rows();
                    const int vals = prob.row_values();
#pragma unroll 1
                    for (int r = 0; r < out_rows && n_cols > 0; ++r) {
                        const uint32_t col = prob.row_column(r);
                        ptx::tmem_ld_32x32(t_row + col, r0);
                        if (vals > 32) ptx::tmem_ld_32x32(t_row + col + 32, r1);
                        ptx::tmem_ld_wait();
                        float v0[32], v1[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            v0[j] = __uint_as_float(r0[j]);
                            v1[j] = __uint_as_float(r1[j]);
                        }
                        prob.finish(tile, row_in_cta, 0, v0, epi);
                        if (vals > 32) prob.finish(tile, row_in_cta, 32, v1, epi);
                        if (lane == 0) ptx::bulk_wait_group_read<0>();      // the previous row's store has read the block
                        __syncwarp();
                        const uint32_t dst = staging + lane * uint32_t(vals) * 4u;
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            if (q * 4 < vals)
                                ptx::st_shared_v4(dst + q * 16, v0[4 * q], v0[4 * q + 1], v0[4 * q + 2], v0[4 * q + 3]);
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            if (32 + q * 4 < vals)
                                ptx::st_shared_v4(dst + 128 + q * 16, v1[4 * q], v1[4 * q + 1], v1[4 * q + 2],
                                                  v1[4 * q + 3]);
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            int x, y, z;
                            prob.row_coords(tile, int(quarter) * 32, r, x, y, z);
                            ptx::tma_store_3d(prob.out_map(), staging, x, y, z);
                            ptx::bulk_commit_group();
                        }
                    }
                }
            } else {
            if (ksplit > 1) {
                // ---- split-K inside the cluster: exchange partial sums, then reduce one slice
                // Exchange buffer: [source group (own one skipped)][32-column chunk of the slice]
                // [16-byte unit of the row (8)][row (128)][16 B]: one store instruction of a warp
                // covers 512 contiguous bytes of the peer's shared memory, and the thread that
                // reduces a row reads back exactly what its counterpart wrote.
                const uint32_t xbuf = smem_base + uint32_t(sched.stages) * STAGE_BYTES;
                const int slice = sched.umma_n / int(ksplit);          // columns this group reduces
                const int slice_chunks = slice / 32;
                const uint32_t row_off = uint32_t(row_in_cta) * 16u;
                // Both loops keep the accumulator load of the next chunk in flight while the current
                // chunk is stored or reduced (two register sets, bodies unrolled twice).
                auto next_foreign = [&](int c) { return (c < n_cols && uint32_t(c / slice) == kgroup) ? c + slice : c; };
                auto send = [&](int c, const uint32_t (&r)[32]) {
                    const uint32_t owner = uint32_t(c / slice);
                    const uint32_t slot = kgroup > owner ? kgroup - 1 : kgroup;
                    const uint32_t chunk = slot * slice_chunks + uint32_t(c - int(owner) * slice) / 32u;
                    const uint32_t dst = ptx::mapa(xbuf + chunk * (UMMA_BM * 128u) + row_off, owner * CTAS + cta_rank);
                    const uint32_t bar = ptx::mapa(ptx::smem_u32(&bar_exchange), owner * CTAS + cta_rank);
#pragma unroll
                    for (uint32_t q = 0; q < 8; ++q)
                        ptx::st_async_v4(dst + q * (UMMA_BM * 16u), r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3],
                                         bar);
                };
                {
                    int c = next_foreign(0);
                    if (c < n_cols) ptx::tmem_ld_32x32(t_row + c, r0);
#pragma unroll 1
                    while (c < n_cols) {
                        ptx::tmem_ld_wait();
                        const int c1 = next_foreign(c + 32);
                        if (c1 < n_cols) ptx::tmem_ld_32x32(t_row + c1, r1);
                        send(c, r0);
                        if (c1 >= n_cols) break;
                        ptx::tmem_ld_wait();
                        c = next_foreign(c1 + 32);
                        if (c < n_cols) ptx::tmem_ld_32x32(t_row + c, r0);
                        send(c1, r1);
                    }
                }
                // This group's own slice does not depend on the others: its first chunk is on its way
                // out of TMEM while the partial sums cross the cluster.
                const int own0 = int(kgroup) * slice;
                if (n_cols > 0) ptx::tmem_ld_32x32(t_row + own0, r0);
                // Nothing to signal: every store counts its own bytes on the owner's barrier when it
                // lands (a release fence and an arrival per warp cost a round trip through the
                // cluster before the arrival could even leave, about 1900 cycles).
                ok = n_cols == 0 || ptx::mbar_wait<true>(ptx::smem_u32(&bar_exchange), 0, wctx, UMMA_TIMEOUT_EXCHANGE);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { ptx::tmem_ld_wait(); break; }
                auto reduce = [&](int cc, uint32_t (&r)[32]) {
                    for (uint32_t slot = 0; slot + 1 < ksplit; ++slot) {      // fixed order: reproducible
                        const uint32_t src = xbuf + (slot * slice_chunks + cc) * (UMMA_BM * 128u) + row_off;
#pragma unroll
                        for (uint32_t q = 0; q < 8; ++q) {
                            const float4 p = ptx::ld_shared_v4(src + q * (UMMA_BM * 16u));
                            r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + p.x);
                            r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + p.y);
                            r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + p.z);
                            r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + p.w);
                        }
                    }
                    // With an output map every chunk of the slice gets a block of its own in the
                    // idle stage ring, and one proxy fence and one group of bulk stores follow the
                    // loop: a fence-and-store round costs about as much for four blocks as for one.
                    if constexpr (Problem::kTmaStore) {
                        if (use_tma) {
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                            prob.finish(tile, row_in_cta, own0 + cc * 32, v, epi);
                            const uint32_t row_smem =
                                smem_base + (quarter * uint32_t(slice_chunks) + uint32_t(cc)) * 4096u + lane * 128u;
#pragma unroll
                            for (uint32_t q = 0; q < 8; ++q)
                                ptx::st_shared_v4(row_smem + ((q ^ (lane & 7u)) << 4), v[4 * q], v[4 * q + 1],
                                                  v[4 * q + 2], v[4 * q + 3]);
                            return;
                        }
                    }
                    emit(own0 + cc * 32, r);
                };
                if (n_cols == 0) ptx::tmem_ld_wait();
#pragma unroll 1
                for (int cc = 0; cc < slice_chunks && n_cols > 0; cc += 2) {
                    ptx::tmem_ld_wait();
                    if (cc + 1 < slice_chunks) ptx::tmem_ld_32x32(t_row + own0 + (cc + 1) * 32, r1);
                    reduce(cc, r0);
                    if (cc + 1 >= slice_chunks) break;
                    ptx::tmem_ld_wait();
                    if (cc + 2 < slice_chunks) ptx::tmem_ld_32x32(t_row + own0 + (cc + 2) * 32, r0);
                    reduce(cc + 1, r1);
                }
                if constexpr (Problem::kTmaStore) {
                    if (use_tma && n_cols > 0) {
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            for (int cc = 0; cc < slice_chunks; ++cc) {
                                int x, y;
                                prob.out_coords(tile, int(quarter) * 32, own0 + cc * 32, x, y);
                                ptx::tma_store_2d(prob.out_map(),
                                                  smem_base + (quarter * uint32_t(slice_chunks) + uint32_t(cc)) * 4096u, x, y);
                            }
                            ptx::bulk_commit_group();
                        }
                    }
                }
            }
            if (ksplit == 1 && use_tma) {
                // Two 32-column chunks per round: both staging blocks are filled, one proxy fence
                // covers them, two bulk stores go out as one group, and the accumulator loads of
                // the next round are in flight while this round is fenced and stored.
                //
                // The CTA's last tile is the one whose epilogue nothing hides.  By then the stage
                // ring is idle (every load was consumed by an MMA that has completed, and the
                // producer has nothing left to issue), so each warp stages all its chunks in a
                // 32 KB slice of the ring, a block per chunk, and never waits for a store to
                // release a block.
                if constexpr (Problem::kTmaStore) {
                    const bool dbg_nold = (sched.debug & 0x20u) != 0, dbg_nost = (sched.debug & 0x10u) != 0;
                    const bool in_ring = sched.ring_staging != 0 && (u + unit_stride >= num_units);
                    uint32_t block0 = in_ring ? smem_base + quarter * 32768u : staging;
                    if (n_cols > 0 && !dbg_nold) ptx::tmem_ld_32x32(t_row, r0);
                    if (n_cols > 32 && !dbg_nold) ptx::tmem_ld_32x32(t_row + 32, r1);
#pragma unroll 1
                    for (int c = 0; c < n_cols; c += 64) {
                        const bool two = c + 32 < n_cols;
                        ptx::tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r0[j]);
                        prob.finish(tile, row_in_cta, c, v, epi);
                        if (!in_ring) {
                            if (lane == 0) ptx::bulk_wait_group_read<0>();  // last round's stores have read their blocks
                            __syncwarp();
                        }
                        const uint32_t row_smem = block0 + lane * 128u;
#pragma unroll
                        for (uint32_t q = 0; q < 8; ++q)      // 128-byte swizzle: unit q of row r at q ^ (r & 7)
                            ptx::st_shared_v4(row_smem + ((q ^ (lane & 7u)) << 4), v[4 * q], v[4 * q + 1],
                                              v[4 * q + 2], v[4 * q + 3]);
                        if (two) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r1[j]);
                            prob.finish(tile, row_in_cta, c + 32, v, epi);
#pragma unroll
                            for (uint32_t q = 0; q < 8; ++q)
                                ptx::st_shared_v4(row_smem + 4096u + ((q ^ (lane & 7u)) << 4), v[4 * q], v[4 * q + 1],
                                                  v[4 * q + 2], v[4 * q + 3]);
                        }
                        if (c + 64 < n_cols && !dbg_nold) ptx::tmem_ld_32x32(t_row + c + 64, r0);
                        if (c + 96 < n_cols && !dbg_nold) ptx::tmem_ld_32x32(t_row + c + 96, r1);
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if constexpr (has_multimem_store<Problem>::value) {
                            int x, y;
                            prob.out_coords(tile, int(quarter) * 32, c, x, y);
                            if (two) prob.multimem_store_pair(block0, x, y, lane);
                            else prob.multimem_store(block0, x, y, lane);
                            __syncwarp();
                        } else if (lane == 0 && !dbg_nost) {
                            int x, y;
                            prob.out_coords(tile, int(quarter) * 32, c, x, y);
                            ptx::tma_store_2d(prob.out_map(), block0, x, y);
                            if (two) ptx::tma_store_2d(prob.out_map(), block0 + 4096u, x + 32, y);
                            push_to_peers(prob, block0, x, y);
                            if (two) push_to_peers(prob, block0 + 4096u, x + 32, y);
                            ptx::bulk_commit_group();
                        }
                        if (in_ring) block0 += 8192u;
                    }
                }
            } else if (ksplit == 1) {
                if (n_cols > 0) ptx::tmem_ld_32x32(t_row, r0);
#pragma unroll 1
                for (int c = 0; c < n_cols; c += 64) {
                    ptx::tmem_ld_wait();
                    if (c + 32 < n_cols) ptx::tmem_ld_32x32(t_row + c + 32, r1);
                    emit(c, r0);
                    if (c + 32 < n_cols) {
                        ptx::tmem_ld_wait();
                        if (c + 64 < n_cols) ptx::tmem_ld_32x32(t_row + c + 64, r0);
                        emit(c + 32, r1);
                    }
                }
            }
            }      // not the row-store form
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                const uint32_t acce_local = ptx::smem_u32(&bar_acc_empty[acc]);
                if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(ptx::mapa(acce_local, leader_rank));
                else ptx::mbar_arrive(acce_local);
            }
        }
        if (CTAS == 2) ptx::cluster_arrive();      // this warp is done with TMEM and with its partner: see the teardown
        // Bulk stores read shared memory asynchronously: the reads must be over before the CTA
        // gives its shared memory back (the writes themselves complete with the kernel).
        if constexpr (has_multimem_store<Problem>::value) __threadfence_system();
        if (lane == 0) {
            if constexpr (has_peer_store<Problem>::value) {
                // Stores into other GPUs' memory: wait for the writes themselves, then order them
                // system-wide before the kernel ends (the peers read C after this launch completes).
                ptx::bulk_wait_group<0>();
                __threadfence_system();
            } else {
                ptx::bulk_wait_group_read<0>();
            }
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // A wait ran out: give copies still in flight a bounded time to land
        // before this CTA's shared memory is handed to the next one.
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    // No CTA of a pair leaves (or frees the pair's TMEM) while its partner may still signal it or
    // read accumulators.  Lone CTAs that only shared a split reduction need no such barrier: each
    // one waited, on its exchange barrier, for everything any other CTA sends it, and the last
    // thing it sent - its arrivals on the others' exchange barriers - is what they wait for.
    // The barrier is split: every warp arrived when its own role ended (the epilogue warps before
    // they waited for their bulk stores to drain), so by now the partner's warps have usually
    // arrived too and the wait costs nothing, instead of a round trip after the drain.
    if (CTAS == 2) ptx::cluster_wait();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
    }
#else
    // Compiled for an architecture without tcgen05: report instead of running.
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(sched.status, 0u, 0xdeadu);
#endif
}

// ---------------------------------------------------------------- host helpers

// A schedule of whole tiles (no K split of either kind, register-store epilogue, no diagnostics)
// for `k_blocks` K blocks per tile; launchers change what they need.
inline UmmaSchedule whole_tile_schedule(int tiles_m, int tiles_n, int k_blocks, int umma_n, uint32_t tx_bytes,
                                        int stages, uint32_t* status_word) {
    UmmaSchedule sched{};
    sched.tiles_m = tiles_m;
    sched.tiles_n = tiles_n;
    sched.k_blocks = k_blocks;
    sched.raster_group = 8;
    sched.status = status_word;
    sched.wait_limit_ns = 2000000000ull;
    sched.umma_n = umma_n;
    sched.tx_bytes = tx_bytes;
    sched.stages = stages;
    sched.n_whole = tiles_m * tiles_n;
    sched.split = 1;
    sched.kb_per_split = k_blocks;
    sched.cluster_split = 1;
    return sched;
}

// Off when the environment variable CUDEEP_B200_PDL is "0" (read once).
bool programmatic_launch_enabled();

// Launches `kernel` on `clusters` clusters of `cluster_size` CTAs with `smem_bytes` of dynamic
// shared memory (the kernel's opt-in limit is raised to `smem_limit` on first use).
template <class Kernel, class Problem>
void launch_umma(Kernel kernel, const Problem& prob, const UmmaSchedule& sched, const UmmaEpilogueArgs& epi,
                 long long clusters, int cluster_size, uint32_t smem_bytes, uint32_t smem_limit,
                 cudaStream_t stream) {
    ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem_limit);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(clusters * cluster_size), 1, 1);
    cfg.blockDim = dim3(UMMA_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int count = 0;
    if (cluster_size > 1) {          // a lone CTA is launched as a plain grid
        attr[count].id = cudaLaunchAttributeClusterDimension;
        attr[count].val.clusterDim.x = unsigned(cluster_size);
        attr[count].val.clusterDim.y = 1;
        attr[count].val.clusterDim.z = 1;
        ++count;
    }
    if (programmatic_launch_enabled()) {
        // The kernel waits for its predecessors itself (grid_dependency_wait), so its set-up may
        // overlap their tail.
        attr[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    cfg.attrs = attr;
    cfg.numAttrs = unsigned(count);
    CB200_CUDA(cudaLaunchKernelEx(&cfg, kernel, prob, sched, epi));
}

}  // namespace cudeep_b200
