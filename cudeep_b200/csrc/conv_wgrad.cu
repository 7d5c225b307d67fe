// grad_weight of a Conv2d as an implicit GEMM on tcgen05
// (reference include/cudeep/kernels/conv.cuh:28-36, src/kernels/conv_kernel.cu:460-545, which
// forms im2col(x) per image in global memory and multiplies it with grad_output).
//
//   dw[oc, c, kh, kw] = sum_{n, oh, ow} dy[n, oc, oh, ow] * x[n, c, oh*sh+kh-ph, ow*sw+kw-pw]
//
// For one filter tap this is D[OC, C] = dY[OC, pixels] * X_tap[pixels, C]: the reduction runs over
// output pixels.  A K block is 32 consecutive pixels of one output row (box_w x box_h = 32 x 1):
//   * A (K-major): grad_output read in place as a 4-D tensor {OW, OH, OC, N}; the box
//     {32, 1, 128, 1} lands as one 128-byte row per output channel;
//     (rows of at most 16 pixels: a copy of grad_output with rows padded to 4, 8 or 16 pixels, whose
//     planes are then contiguous runs of OH * pitch floats, so that 32 consecutive floats of a plane
//     are 32 / pitch whole rows - box_w x box_h = pitch x 32 / pitch - and a 7 x 7 feature map fills
//     28 of a block's 32 pixels instead of 7);
//   * B (MN-major, channels contiguous): the NHWC copy of the input (channels padded to 32) seen
//     as a 5-D tensor {32, W, H, N, Cp/32}; the box {32, box_w, box_h, 1, chunks}, started at the
//     tap's offset, lands as 32-channel chunks of 32 pixel rows - the layout the tensor core takes
//     for an MN-major 32-bit operand.  Padding is the out-of-range zero fill of either side.
// Nothing of size pixels x C*KH*KW is written.  There are only taps * ceil(C / 256) output tiles
// per 256 output channels but a very long K, so K is cut into ranges, one tile-sized partial
// result per range goes to scratch (bulk tensor stores), and a small kernel adds the ranges in a
// fixed order and writes the [OC][C][KH][KW] layout - bitwise reproducible, no atomics.
#include <cstdlib>

#include "conv_igemm.h"
#include "umma_gemm.cuh"

namespace cudeep_b200 {

namespace {

// ROW_PACKED (few input channels): one tile per filter row instead of per tap; map_x is the view
// {KW * Cx, OW, H, N, 1} of the width-padded input copy, whose rows are the windows of KW pixels x Cx
// channels the output columns read (the forward path's row-packed form), so the 32 columns of a
// tile are a filter row's (tap, channel) pairs.
// TAP_SHIFT (one CTA per tile, stride 1, three taps per filter row, rows of more than 16 pixels): a
// tile is one filter row kh and 64 channels; its 192 accumulator columns are [kw][channel], and the
// K step loads 32 + 4 input pixels once for the three taps (tap_shift_of in umma_gemm.cuh).
template <int CTAS, bool ROW_PACKED = false, bool MULTI_TAP = false, bool TAP_SHIFT = false>
struct WgradProblem {
    static constexpr bool kTmaStore = true;
    static constexpr bool kClusterSplit = false;
    static constexpr int kTapShift = TAP_SHIFT ? 3 : 0;
    static constexpr int kTapColumns = 64;
    CUtensorMap map_dy;     // {OW, OH, OC, N}, box {box_w, box_h, 128, 1}
    CUtensorMap map_x;      // {32, W, H, N, Cp/32}, box {32, box_w, box_h, 1, chunks per CTA}
    CUtensorMap map_part;   // partial results [ranges * OCp][taps * Cp], box {32, 32}
    int tiles_w, tiles_h;   // pixel boxes per image
    int box_w, box_h;
    int c_tiles;            // channel tiles (of umma_n channels) per tap
    int taps, k_w, p_h, p_w;
    int s_h, s_w;           // convolution strides
    int n_cols;             // accumulator columns per tile (umma_n)
    int taps_per_tile;      // > 1 (few channels): a tile's columns are this many taps x all cp channels, so the
                            // grad_output block a K step loads serves several taps (c_tiles == 1 then)
    int cp;                 // padded channels
    int ocp;                // padded output channels: rows of one K range in the scratch
    int dy_row_pitch;       // > 0: map_dy is {OH * pitch, 1, OC, N} over a copy with rows padded to `pitch`
    int kb_per_range;       // K blocks (pixel boxes) of one range
    int total_kb;           // batch * tiles_h * tiles_w
    int batch;

    struct Tile {
        int oc0;            // first output channel of this CTA
        int tap, c0;        // filter tap and first channel of the tile
        int cb0;            // first channel this CTA stages
        int range;          // which K range
    };

    __device__ __forceinline__ void prefetch_maps() const {
        ptx::prefetch_tensormap(&map_dy);
        ptx::prefetch_tensormap(&map_x);
        ptx::prefetch_tensormap(&map_part);
    }
    // tn enumerates (range, tap, channel tile), the channel tile fastest.
    __device__ __forceinline__ Tile decode(int tm, int tn, uint32_t cta_rank) const {
        Tile t;
        t.oc0 = (tm * CTAS + int(cta_rank)) * UMMA_BM;
        const int tap_tiles = (taps + taps_per_tile - 1) / taps_per_tile;
        const int per_range = tap_tiles * c_tiles;
        t.range = tn / per_range;
        const int r = tn - t.range * per_range;
        const int tap_tile = r / c_tiles;
        t.tap = tap_tile * taps_per_tile;
        if constexpr (TAP_SHIFT) {
            // tn enumerates (range, kh, 64-channel tile); t.tap is the row's first tap.
            const int c64 = cp / 64;
            const int kh = r / c64;
            t.tap = kh * k_w;
            t.c0 = (r - kh * c64) * 64;
            t.cb0 = t.c0;
        } else if constexpr (MULTI_TAP) {
            // cb0: the first of the tile's taps this CTA stages (all channels of each).
            t.c0 = 0;
            t.cb0 = int(cta_rank) * (taps_per_tile / CTAS);
        } else {
            t.c0 = (r - tap_tile * c_tiles) * n_cols;
            t.cb0 = t.c0 + int(cta_rank) * (n_cols / CTAS);
        }
        return t;
    }
    template <int C>
    __device__ __forceinline__ void load(const Tile& t, int kb, uint32_t a_smem, uint32_t b_smem,
                                         uint32_t bar) const {
        const int g = t.range * kb_per_range + kb;      // pixel box over the whole batch
        const int per_image = tiles_h * tiles_w;
        // Blocks past the end of this range or of the batch read zeros on both sides: the
        // image index is pushed out of range.
        int n = g / per_image;
        const int r = g - n * per_image;
        if (kb >= kb_per_range || g >= total_kb) n = batch;
        const int th = r / tiles_w;
        const int oh0 = th * box_h;
        const int ow0 = (r - th * tiles_w) * box_w;
        const int dy_x = dy_row_pitch > 0 ? oh0 * dy_row_pitch : ow0;
        const int dy_y = dy_row_pitch > 0 ? 0 : oh0;
        if constexpr (C == 1) ptx::tma_load_4d(a_smem, &map_dy, bar, dy_x, dy_y, t.oc0, n);
        else ptx::tma_load_4d_pair(a_smem, &map_dy, bar, dy_x, dy_y, t.oc0, n);
        if constexpr (TAP_SHIFT) {
            // The pixels under filter row kh for all three taps: 36 from the first tap's start on.
            const int kh = t.tap / k_w;
            ptx::tma_load_5d(b_smem, &map_x, bar, 0, ow0 - p_w, oh0 + kh - p_h, n, t.cb0 / 32);
            return;
        }
        if constexpr (MULTI_TAP) {
            {
                // One box of all channels per tap, side by side as column groups; a tap past the
                // filter's last one reads zeros (image index out of range), its columns are clipped.
                const int mine = taps_per_tile / C;
                const uint32_t group_bytes = uint32_t(cp / 32) * 4096u;
                for (int tl = 0; tl < mine; ++tl) {
                    const int tap = t.tap + t.cb0 + tl;
                    const int kh = tap / k_w;
                    const int x1 = ow0 * s_w + (tap - kh * k_w) - p_w;
                    const int nn = tap < taps ? n : batch;
                    if constexpr (C == 1)
                        ptx::tma_load_5d(b_smem + tl * group_bytes, &map_x, bar, 0, x1, oh0 * s_h + kh - p_h, nn, 0);
                    else
                        ptx::tma_load_5d_pair(b_smem + tl * group_bytes, &map_x, bar, 0, x1, oh0 * s_h + kh - p_h, nn, 0);
                }
                return;
            }
        }
        const int kh = ROW_PACKED ? t.tap : t.tap / k_w;
        const int x1 = ROW_PACKED ? ow0 : ow0 * s_w + (t.tap - kh * k_w) - p_w;
        if constexpr (C == 1) ptx::tma_load_5d(b_smem, &map_x, bar, 0, x1, oh0 * s_h + kh - p_h, n, t.cb0 / 32);
        else ptx::tma_load_5d_pair(b_smem, &map_x, bar, 0, x1, oh0 * s_h + kh - p_h, n, t.cb0 / 32);
    }
    __device__ __forceinline__ const CUtensorMap* out_map() const { return &map_part; }
    __device__ __forceinline__ void out_coords(const Tile& t, int row_in_cta, int c0, int& x, int& y) const {
        if constexpr (TAP_SHIFT) x = (t.tap + c0 / 64) * cp + t.c0 + (c0 & 63);      // columns are [kw][64 channels]
        else x = t.tap * cp + t.c0 + c0;
        y = t.range * ocp + t.oc0 + row_in_cta;
    }
    __device__ __forceinline__ void finish(const Tile&, int, int, float (&)[32], const UmmaEpilogueArgs&) const {}
    // Every tile goes out through the bulk-store path.
    __device__ __forceinline__ void store(const Tile&, int, int, float (&)[32], const UmmaEpilogueArgs&, int) const {}
};

// Copies rows of `ow` floats to rows of `pitch` floats (pitch >= ow, a multiple of 4), zero in
// the tail: grad_output with 16-byte-aligned rows for the tensor map.
__global__ void pad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, long long rows, int ow,
                                int pitch) {
    // One 128-bit store per thread; 32-bit index arithmetic (the launcher checks the range).
    const unsigned quads = static_cast<unsigned>(pitch / 4);
    const unsigned total = static_cast<unsigned>(rows) * quads;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const unsigned r = i / quads;
        const int q = static_cast<int>(i - r * quads) * 4;
        const float* row = src + static_cast<long long>(r) * ow;
        float4 v;
        v.x = q + 0 < ow ? row[q + 0] : 0.0f;
        v.y = q + 1 < ow ? row[q + 1] : 0.0f;
        v.z = q + 2 < ow ? row[q + 2] : 0.0f;
        v.w = q + 3 < ow ? row[q + 3] : 0.0f;
        reinterpret_cast<float4*>(dst)[i] = v;
    }
}

// dw[oc][c][tap] = sum over ranges of part[range][oc][tap * cp + c], ranges in ascending order.
// A block takes one output channel and a chunk of channels with all their taps: it reads the
// partial tiles along c, 128 bits per thread and range (few values per thread, so the bytes in
// flight are what sets the speed), keeps the sums in shared memory as [tap][chunk + 4] and writes
// its part of dw, which is one run of consecutive floats.
constexpr int kReduceTile = 3072;
__global__ void __launch_bounds__(256)
wgrad_reduce_kernel(const float* __restrict__ part, float* __restrict__ dw, int ranges, int oc_n, int ocp,
                    int c_n, int cp, int taps, int chunk) {
    __shared__ __align__(16) float tile[kReduceTile];
    const int chunks = (c_n + chunk - 1) / chunk;
    const long long units = static_cast<long long>(oc_n) * chunks;
    const long long row_len = static_cast<long long>(taps) * cp;
    const long long range_stride = static_cast<long long>(ocp) * row_len;
    const int pitch = chunk + 4;
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const long long oc = u / chunks;
        const int c0 = static_cast<int>(u - oc * chunks) * chunk;
        const int width = min(chunk, c_n - c0);
        const int quads = (width + 3) / 4;          // columns up to cp exist in the partial tiles (zeros past C)
        const float* src = part + oc * row_len + c0;
        for (int i = threadIdx.x; i < quads * taps; i += blockDim.x) {
            const int tap = i / quads, q4 = i - tap * quads;
            const float4* q = reinterpret_cast<const float4*>(src + static_cast<long long>(tap) * cp) + q4;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
            for (int s = 0; s < ranges; ++s) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q) + s * range_stride));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            *reinterpret_cast<float4*>(&tile[tap * pitch + 4 * q4]) = acc;
        }
        __syncthreads();
        float* dst = dw + (oc * c_n + c0) * taps;
        for (int i = threadIdx.x; i < width * taps; i += blockDim.x) {
            const int cc = i / taps, tap = i - cc * taps;
            dst[i] = tile[tap * pitch + cc];
        }
        __syncthreads();
    }
}

// The same sum for filters with more than 65 taps (a chunk of 32 channels would not fit the tile):
// threads walk (oc, tap, c) with c fastest, so the reads coalesce; the writes are strided by the
// tap count.
__global__ void wgrad_reduce_wide_kernel(const float* __restrict__ part, float* __restrict__ dw, int ranges,
                                         int oc_n, int ocp, int c_n, int cp, int taps) {
    const long long total = static_cast<long long>(oc_n) * taps * c_n;
    const long long row_len = static_cast<long long>(taps) * cp;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % c_n);
        const long long r = i / c_n;
        const int tap = static_cast<int>(r % taps);
        const long long oc = r / taps;
        const float* src = part + oc * row_len + static_cast<long long>(tap) * cp + c;
        float acc = 0.0f;
        for (int s = 0; s < ranges; ++s) acc += src[static_cast<long long>(s) * ocp * row_len];
        dw[(oc * c_n + c) * taps + tap] = acc;
    }
}

// Row-packed tiles: dw[oc][c][kh][kw] = sum over ranges of part[range][oc][kh * 32 + kw * cx + c].
__global__ void wgrad_reduce_rows_kernel(const float* __restrict__ part, float* __restrict__ dw, int ranges,
                                         int oc_n, int ocp, int c_n, int cx, int k_h, int k_w) {
    const long long total = static_cast<long long>(oc_n) * c_n * k_h * k_w;
    const long long row_len = static_cast<long long>(k_h) * UMMA_BK;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int kw = static_cast<int>(i % k_w);
        long long r = i / k_w;
        const int kh = static_cast<int>(r % k_h);
        r /= k_h;
        const int c = static_cast<int>(r % c_n);
        const long long oc = r / c_n;
        const float* src = part + oc * row_len + kh * UMMA_BK + kw * cx + c;
        float acc = 0.0f;
        for (int s = 0; s < ranges; ++s) acc += src[static_cast<long long>(s) * ocp * row_len];
        dw[i] = acc;
    }
}

struct WgradPlan {
    bool row_packed;    // few input channels: one tile per filter row
    int taps;           // tiles per channel tile: KH * KW, or KH when row-packed
    int dy_pitch;       // floats per row of the grad_output the kernel reads
    bool narrow;        // rows of at most 16 pixels: several rows per K block, always from a padded copy
    int ctas, box_w, box_h, n_cols, c_tiles, ranges, kb_per_range, tiles_w, tiles_h, cp, ocp;
    int taps_per_tile;  // see WgradProblem
    bool tap_shift;     // one load of the input pixels serves the three taps of a filter row
    size_t nhwc_bytes, part_bytes;
};

int round_up(int v, int m) { return (v + m - 1) / m * m; }

WgradPlan plan_wgrad(const ConvShape& s, int num_sms) {
    WgradPlan p{};
    const int oh = s.out_h(), ow = s.out_w();
    p.ctas = s.out_c > UMMA_BM ? 2 : 1;
    p.cp = round_up(s.in_c, UMMA_BK);
    p.row_packed = conv2d_igemm_row_packed(s);
    p.taps = p.row_packed ? s.k_h : s.k_h * s.k_w;
    // Channels per tile: the widest multiple of one 32-channel chunk per CTA, at most 256, that
    // divides the padded channel count (a tile never reaches into the next tap's columns).
    auto widest = [&](int step) {
        for (int n = 256; n >= step; n -= step)
            if (n % step == 0 && p.cp % n == 0) return n;
        return 0;
    };
    p.n_cols = widest(32 * p.ctas);
    if (p.ctas == 2 && p.n_cols < 128) {
        p.ctas = 1;
        p.n_cols = widest(32);
    }
    p.c_tiles = p.cp / p.n_cols;
    // Few channels: the accumulator's 256 columns hold several taps of all channels, so that the
    // grad_output block of a K step (128 requests of the TMA unit, whatever the channel count) is
    // multiplied with 256 columns instead of 64 or 128.
    p.taps_per_tile = 1;
    static const bool several_taps = [] { const char* v = std::getenv("CUDEEP_B200_WGRAD_TAPS"); return !(v && v[0] == '0'); }();
    if (several_taps && !p.row_packed && p.cp <= 128 && p.taps >= 2) {
        // How many: the count (even for a pair, which splits the taps between its CTAs) that needs the
        // fewest requests for all taps - per tile and K step 128 rows of grad_output and one row of
        // 32 pixels per channel chunk and tap.  A 3 x 3 filter over 64 channels takes 3 tiles of
        // 3 taps (192 columns), not 2 of 4 and one of 1.
        p.ctas = s.out_c > UMMA_BM ? 2 : 1;           // 128 columns per CTA of a pair again
        long long best_cost = -1;
        for (int t = p.ctas; t * p.cp <= 256; t += p.ctas) {
            const long long cost = static_cast<long long>((p.taps + t - 1) / t) * (128 + t * p.cp);
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                p.taps_per_tile = t;
            }
        }
        p.n_cols = p.taps_per_tile * p.cp;
        p.c_tiles = 1;
        if (p.taps_per_tile == 1) p.n_cols = p.cp;    // (a pair never gets here: its smallest count is 2)
    }
    // One CTA per tile, stride 1, three taps per filter row, whole 64-channel tiles: the taps share the pixels.
    p.tap_shift = several_taps && !p.row_packed && s.out_c <= UMMA_BM && s.k_w == 3 && s.s_h == 1 && s.s_w == 1 &&
                  p.cp % 64 == 0 && ow > 16;
    if (p.tap_shift) {
        p.ctas = 1;
        p.taps_per_tile = 3;
        p.n_cols = 192;
        p.c_tiles = p.cp / 64;
    }
    // A K block is 32 consecutive pixels of one output row.  A swizzled TMA box whose inner extent
    // is under 128 bytes is not packed densely in shared memory, so boxes of 16 x 2 or 8 x 4 pixels
    // cannot be read from grad_output in place; for rows of at most 16 pixels they are read from
    // a copy whose rows are padded to 4, 8 or 16, as 32 consecutive floats of a plane.
    p.narrow = ow <= 16;
    p.dy_pitch = round_up(ow, 4);
    p.box_w = 32;
    p.box_h = 1;
    if (p.narrow) {
        p.dy_pitch = ow <= 4 ? 4 : ow <= 8 ? 8 : 16;
        p.box_w = p.dy_pitch;
        p.box_h = 32 / p.dy_pitch;
    }
    p.tiles_w = (ow + p.box_w - 1) / p.box_w;
    p.tiles_h = (oh + p.box_h - 1) / p.box_h;
    const long long total_kb = static_cast<long long>(s.batch) * p.tiles_h * p.tiles_w;
    const int tiles_m = (s.out_c + UMMA_BM * p.ctas - 1) / (UMMA_BM * p.ctas);
    p.ocp = tiles_m * UMMA_BM * p.ctas;
    const int tap_tiles = (p.taps + p.taps_per_tile - 1) / p.taps_per_tile;
    const long long base_tiles = static_cast<long long>(tiles_m) * tap_tiles * p.c_tiles;
    // Enough K ranges to give every CTA (pair) a unit, each at least 16 K blocks long.
    const long long slots = num_sms / p.ctas;
    long long ranges = slots / base_tiles;
    if (ranges > total_kb / 16) ranges = total_kb / 16;
    if (ranges < 1) ranges = 1;
    if (ranges > 64) ranges = 64;
    long long per = (total_kb + ranges - 1) / ranges;
    per = (per + 1) / 2 * 2;                              // whole pipeline stages of two K blocks
    p.kb_per_range = static_cast<int>(per);
    p.ranges = static_cast<int>((total_kb + per - 1) / per);
    const size_t nhwc = p.row_packed
        ? static_cast<size_t>(s.batch) * s.in_h * (s.in_w + 2 * s.p_w) * round_up(s.in_c, 4) * sizeof(float)
        : static_cast<size_t>(s.batch) * s.in_h * s.in_w * p.cp * sizeof(float);
    p.nhwc_bytes = (nhwc + 1023) / 1024 * 1024;
    p.part_bytes = static_cast<size_t>(p.ranges) * p.ocp * p.taps * p.cp * sizeof(float);
    return p;
}

// dy_pitch: floats between consecutive rows of grad_output as passed here (OW, or the plan's
// pitch when a padded copy had to be made).
template <int CTAS, int KATOMS, bool ROW_PACKED = false, bool MULTI_TAP = false, bool TAP_SHIFT = false>
void launch_wgrad(const float* dy, int dy_pitch, const float* xt, float* part, const ConvShape& s,
                  const WgradPlan& p, cudaStream_t stream) {
    using Cfg = UmmaConfig<CTAS, 256, true, KATOMS>;
    using Prob = WgradProblem<CTAS, ROW_PACKED, MULTI_TAP, TAP_SHIFT>;
    const DeviceInfo& dev = device_info();
    const int oh = s.out_h(), ow = s.out_w();
    const int taps = p.taps;

    Prob prob;
    if (p.narrow) {
        const uint64_t plane = uint64_t(oh) * dy_pitch;
        const uint64_t dims[4] = {plane, 1, uint64_t(s.out_c), uint64_t(s.batch)};
        const uint64_t strides[3] = {plane * 4, plane * 4, uint64_t(s.out_c) * plane * 4};
        const uint32_t box[4] = {32, 1, UMMA_BM, 1};
        encode_tensor_map(&prob.map_dy, dy, 4, dims, strides, box, TmaSwizzle::B128);
    } else {
        const uint64_t dims[4] = {uint64_t(ow), uint64_t(oh), uint64_t(s.out_c), uint64_t(s.batch)};
        const uint64_t strides[3] = {uint64_t(dy_pitch) * 4, uint64_t(oh) * dy_pitch * 4,
                                     uint64_t(s.out_c) * oh * dy_pitch * 4};
        const uint32_t box[4] = {uint32_t(p.box_w), uint32_t(p.box_h), UMMA_BM, 1};
        encode_tensor_map(&prob.map_dy, dy, 4, dims, strides, box, TmaSwizzle::B128);
    }
    if (ROW_PACKED) {
        const int cx = round_up(s.in_c, 4);
        const uint64_t wp_pixels = uint64_t(s.in_w) + 2 * s.p_w;
        const uint64_t dims[5] = {uint64_t(s.k_w) * cx, uint64_t(ow), uint64_t(s.in_h), uint64_t(s.batch), 1};
        const uint64_t strides[4] = {uint64_t(s.s_w) * cx * 4, wp_pixels * cx * 4,
                                     uint64_t(s.in_h) * wp_pixels * cx * 4, 128};
        const uint32_t box[5] = {32, uint32_t(p.box_w), uint32_t(p.box_h * s.s_h), 1, 1};
        const uint32_t steps[5] = {1, 1, uint32_t(s.s_h), 1, 1};
        encode_tensor_map(&prob.map_x, xt, 5, dims, strides, box, TmaSwizzle::B128Atom32, steps);
    } else {
        const uint64_t dims[5] = {32, uint64_t(s.in_w), uint64_t(s.in_h), uint64_t(s.batch), uint64_t(p.cp / 32)};
        const uint64_t strides[4] = {uint64_t(p.cp) * 4, uint64_t(s.in_w) * p.cp * 4,
                                     uint64_t(s.in_h) * s.in_w * p.cp * 4, 128};
        // With strides the box spans box * stride input pixels walked in steps of the stride.
        // (Tap shift: 32 pixels and the next 4, of which the taps reach 2; 36 rows keep every
        // 32-channel chunk on a 512-byte boundary, the period of the swizzle.  Two chunks per tile.)
        const uint32_t box[5] = {32, uint32_t(TAP_SHIFT ? 36 : p.box_w * s.s_w), uint32_t(p.box_h * s.s_h), 1,
                                 uint32_t(TAP_SHIFT ? 2 : p.taps_per_tile > 1 ? p.cp / 32 : p.n_cols / CTAS / 32)};
        const uint32_t steps[5] = {1, uint32_t(s.s_w), uint32_t(s.s_h), 1, 1};
        encode_tensor_map(&prob.map_x, xt, 5, dims, strides, box, TmaSwizzle::B128Atom32, steps);
    }
    {
        const uint64_t dims[2] = {uint64_t(taps) * p.cp, uint64_t(p.ranges) * p.ocp};
        const uint64_t strides[1] = {uint64_t(taps) * p.cp * 4};
        const uint32_t box[2] = {32, 32};
        encode_tensor_map(&prob.map_part, part, 2, dims, strides, box, TmaSwizzle::B128);
    }
    prob.tiles_w = p.tiles_w;
    prob.tiles_h = p.tiles_h;
    prob.box_w = p.box_w;
    prob.box_h = p.box_h;
    prob.c_tiles = p.c_tiles;
    prob.taps = taps;
    prob.k_w = s.k_w;
    prob.p_h = s.p_h;
    prob.p_w = s.p_w;
    prob.s_h = s.s_h;
    prob.s_w = s.s_w;
    prob.n_cols = p.n_cols;
    prob.taps_per_tile = p.taps_per_tile;
    prob.cp = p.cp;
    prob.ocp = p.ocp;
    prob.dy_row_pitch = p.narrow ? dy_pitch : 0;
    prob.kb_per_range = p.kb_per_range;
    prob.total_kb = s.batch * p.tiles_h * p.tiles_w;
    prob.batch = s.batch;

    const int fit_stages = int((Cfg::SMEM_BUDGET - UMMA_STORE_STAGING_BYTES) / Cfg::STAGE_BYTES);
    UmmaSchedule sched = whole_tile_schedule(
        p.ocp / (UMMA_BM * CTAS), p.ranges * ((taps + p.taps_per_tile - 1) / p.taps_per_tile) * p.c_tiles,
        p.kb_per_range, p.n_cols,
        TAP_SHIFT ? Cfg::A_BYTES + 2u * 36u * 128u : (Cfg::A_BYTES + uint32_t(p.n_cols / CTAS) * UMMA_BK * 4) * CTAS * KATOMS,
        fit_stages < Cfg::STAGES ? fit_stages : Cfg::STAGES, dev.status_word);
    sched.raster_group = sched.tiles_m;
    if (TAP_SHIFT) sched.b_lbo = 36u * 128u;      // channel chunks lie one 36-row box apart
    sched.tma_store = 1;
    sched.ring_staging = uint32_t(sched.stages) * Cfg::STAGE_BYTES >= 131072u ? 1 : 0;
    const uint32_t smem_bytes = uint32_t(sched.stages) * Cfg::STAGE_BYTES + UMMA_STORE_STAGING_BYTES + 1024;

    const long long num_tiles = static_cast<long long>(sched.tiles_m) * sched.tiles_n;
    long long groups = dev.num_sms / CTAS;
    if (groups < 1) groups = 1;
    if (groups > num_tiles) groups = num_tiles;

    CB200_TRACE("conv2d grad_weight implicit GEMM tcgen05: N=%d C=%d %dx%d OC=%d, %dx%d stride %dx%d; %d columns, "
                "taps per tile=%d%s, K ranges=%d of %d blocks, ctas/mma=%d stages=%d clusters=%lld",
                s.batch, s.in_c, s.in_h, s.in_w, s.out_c, s.k_h, s.k_w, s.s_h, s.s_w, p.n_cols, p.taps_per_tile,
                TAP_SHIFT ? " sharing one load of the pixels" : "", p.ranges, p.kb_per_range, CTAS, sched.stages, groups);
    auto kernel = umma_tf32_kernel<CTAS, 256, true, KATOMS, Prob>;
    UmmaEpilogueArgs epi{nullptr, 0, EPI_NONE};
    launch_umma(kernel, prob, sched, epi, groups, CTAS, smem_bytes, Cfg::SMEM_MAX, stream);
}

}  // namespace

bool conv2d_wgrad_igemm_supported(const ConvShape& s) {
    if (device_info().cc_major != 10) return false;
    if (s.s_h < 1 || s.s_w < 1 || s.s_h > 8 || s.s_w > 8) return false;     // 32 pixels x stride <= 256, TMA steps <= 8
    if (s.p_h >= s.k_h || s.p_w >= s.k_w) return false;     // keeps every box start within TMA's signed range
    const int oh = s.out_h(), ow = s.out_w();
    if (oh < 1 || ow < 1) return false;
    if (s.out_c < 32) return false;
    if (static_cast<long long>(s.batch) * oh * ow < 256) return false;
    return true;
}

void conv2d_wgrad_igemm(const float* grad_output, const float* input, float* grad_weight, const ConvShape& s,
                        cudaStream_t stream) {
    check_conv_shape(s);
    CB200_REQUIRE(conv2d_wgrad_igemm_supported(s), "conv2d backward: shape not supported by the tensor-core path");
    const WgradPlan p = plan_wgrad(s, device_info().num_sms);
    // The tensor map of grad_output needs 16-byte-aligned rows: when OW is not a multiple of 4 (14 x 14
    // and 7 x 7 feature maps) or the pointer is unaligned, a padded copy is read instead.
    const int oh = s.out_h(), ow = s.out_w();
    const int dy_pitch = p.dy_pitch;
    const bool copy_dy = ow != dy_pitch || (reinterpret_cast<uintptr_t>(grad_output) & 15u) != 0;
    const size_t part_bytes = (p.part_bytes + 1023) / 1024 * 1024;
    const size_t dy_bytes = copy_dy ? static_cast<size_t>(s.batch) * s.out_c * oh * dy_pitch * sizeof(float) : 0;
    char* scratch = static_cast<char*>(scratch_alloc(p.nhwc_bytes + part_bytes + dy_bytes, stream));
    try {
        float* xt = reinterpret_cast<float*>(scratch);
        float* part = reinterpret_cast<float*>(scratch + p.nhwc_bytes);
        const float* dy = grad_output;
        if (copy_dy) {
            float* padded = reinterpret_cast<float*>(scratch + p.nhwc_bytes + part_bytes);
            const long long rows = static_cast<long long>(s.batch) * s.out_c * oh;
            CB200_REQUIRE(rows * (dy_pitch / 4) < (1LL << 31), "conv2d backward: grad_output too large to pad");
            long long blocks = (rows * (dy_pitch / 4) + 255) / 256;
            if (blocks > 148 * 16) blocks = 148 * 16;
            pad_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(grad_output, padded, rows, ow, dy_pitch);
            CB200_CHECK_LAUNCH();
            dy = padded;
        }
        const long long total = static_cast<long long>(s.out_c) * s.in_c * s.k_h * s.k_w;
        long long blocks = (total + 255) / 256;
        if (blocks > 4096) blocks = 4096;
        if (p.row_packed) {
            const int cx = round_up(s.in_c, 4);
            nchw_to_nhwc_padded(input, xt, s.batch, s.in_c, s.in_h, s.in_w, cx, s.p_w, stream);
            launch_wgrad<1, 1, true>(dy, copy_dy ? dy_pitch : ow, xt, part, s, p, stream);
            wgrad_reduce_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
                part, grad_weight, p.ranges, s.out_c, p.ocp, s.in_c, cx, s.k_h, s.k_w);
        } else {
            nchw_to_nhwc(input, xt, s.batch, s.in_c, s.in_h * s.in_w, p.cp, stream);
            const int pitch = copy_dy ? dy_pitch : ow;
            if (p.tap_shift) {
                launch_wgrad<1, 1, false, false, true>(dy, pitch, xt, part, s, p, stream);
            } else if (p.taps_per_tile > 1) {
                if (p.ctas == 2) launch_wgrad<2, 2, false, true>(dy, pitch, xt, part, s, p, stream);
                else launch_wgrad<1, 1, false, true>(dy, pitch, xt, part, s, p, stream);
            } else if (p.ctas == 2) {
                launch_wgrad<2, 2>(dy, pitch, xt, part, s, p, stream);
            } else {
                launch_wgrad<1, 1>(dy, pitch, xt, part, s, p, stream);
            }
            const int taps = s.k_h * s.k_w;
            if (taps <= 65) {
                // Channels per block: as many 32-channel groups as fit the tile (all of them for 1 x 1).
                int chunk = (kReduceTile / taps - 4) / 32 * 32;
                if (chunk > p.cp) chunk = p.cp;
                long long units = static_cast<long long>(s.out_c) * ((s.in_c + chunk - 1) / chunk);
                if (units > 148 * 16) units = 148 * 16;
                wgrad_reduce_kernel<<<static_cast<unsigned>(units), 256, 0, stream>>>(
                    part, grad_weight, p.ranges, s.out_c, p.ocp, s.in_c, p.cp, taps, chunk);
            } else {
                wgrad_reduce_wide_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
                    part, grad_weight, p.ranges, s.out_c, p.ocp, s.in_c, p.cp, taps);
            }
        }
        CB200_CHECK_LAUNCH();
    } catch (...) {
        scratch_free(scratch, stream);
        throw;
    }
    scratch_free(scratch, stream);
}

}  // namespace cudeep_b200
