// Conv2d forward as an implicit GEMM on tcgen05.
//
//   out[n, oc, oh, ow] = act( sum_{kh,kw,c} w[oc, c, kh, kw] * x[n, c, oh*sh+kh-ph, ow*sw+kw-pw] + bias[oc] )
//
// is computed as D[OC, pixels] = Wp[OC, K] * X[K, pixels] with K ordered
// (kh, kw, c).  Nothing of size K x pixels is ever written to memory:
//   * filters are packed once per call to Wp[OC][KH*KW][Cp] (Cp = C rounded up
//     to 32, zero filled), a K-major A operand;
//   * the input is re-laid once per call as NHWC (channels padded to a
//     multiple of 4).  A K block is then "32 channels of one filter tap", and
//     the B tile of a block of output pixels is a 4-D TMA box
//     {32 channels, box_w, box_h, 1 image} whose start coordinate carries the
//     tap offset (ow0*sw+kw-pw, oh0*sh+kh-ph); padding is TMA's out-of-range zero
//     fill, and a strided convolution's every s-th pixel is the TMA box's element
//     stride.  The box lands in shared memory as one 128-byte row per pixel,
//     which is a K-major B operand as is.
// Accumulator rows are output channels and columns are output pixels, so the
// epilogue writes NCHW directly with bias and activation fused.
//
// The reference takes this shape through Winograd F(4,3) with three global
// temporaries and 36 GEMMs, or through im2col + GEMM + transpose
// (src/kernels/conv_kernel.cu:225-335, :735-789).
#include "conv_igemm.h"
#include "umma_gemm.cuh"

#include <cstdlib>
#include <vector>

namespace cudeep_b200 {

namespace {

// ------------------------------------------------------------------ layout transforms

inline int round_up_int(int v, int m) { return (v + m - 1) / m * m; }

// Filters -> wp[OC][KH*KW][Cp], the K-major A operand (zero for c >= C); OC and C are the output and
// input channel counts of the convolution being launched.
//   plain:   w is [OC][C][KH][KW]:  wp[oc][kh*KW + kw][c] = w[oc][c][kh][kw];
//   flipped: the launch computes a grad_input, whose filters are the forward ones with both
//            spatial axes reversed and the channel axes swapped; w is the forward tensor, which
//            in this launch's terms is [C][OC][KH][KW]:
//            wp[oc][kh*KW + kw][c] = w[c][oc][KH-1-kh][KW-1-kw].
//   row-packed (row_cx > 0, few input channels): one 32-wide K block per filter row holds its
//            KW taps of row_cx channels each, wp[oc][kh][kw * row_cx + c] = w[oc][c][kh][kw].
//   parity classes (sub_sh > 0): the launch computes the grad_input of a strided layer as one
//            stride-1 convolution whose output channels are (class, forward input channel) pairs,
//            oc = (a * sub_sw + b) * fwd_c + ci.  Tap (kh, kw) of the launch is tap
//            j = pad_h - kh + lo_h[a], l = pad_w - kw + lo_w[b] of class (a, b)'s sub-filter, i.e.
//            forward tap (a + sub_sh * j, b + sub_sw * l), and zero where that tap does not exist:
//            wp[oc][kh*KW + kw][c] = w[c][ci][a + sub_sh*j][b + sub_sw*l].
// Eight small signed integers in one word, read by shifting.  (An array member indexed at run
// time makes the compiler keep a copy of the whole kernel-parameter struct in local memory, which
// every thread of the kernel then fills on entry: that doubled the time of the re-layout kernel.)
struct PackedInts8 {
    unsigned long long bits = 0;
    __host__ __device__ void set(int i, int v) {
        bits = (bits & ~(0xffull << (8 * i))) |
               (static_cast<unsigned long long>(static_cast<unsigned char>(static_cast<signed char>(v))) << (8 * i));
    }
    __host__ __device__ int operator[](int i) const { return static_cast<signed char>(bits >> (8 * i)); }
};

struct FilterPack {
    const float* w;
    float* wp;
    int oc_n, c, k_h, k_w, cp, flipped, row_cx;
    int sub_sh = 0, sub_sw = 0, fwd_c = 0, full_kh = 0, full_kw = 0, pad_h = 0, pad_w = 0;
    PackedInts8 lo_h, lo_w;
};

// `tile`: 32 x 65 floats of shared memory, or nullptr.  With it the plain and the flipped form go
// through shared memory so that both the reads and the writes are runs of consecutive floats (the
// direct loop below reads one float per KH * KW of them, or per C * KH * KW when flipped).
__device__ __forceinline__ void pack_filters(const FilterPack& f, long long block, long long blocks, int threads,
                                             float* tile = nullptr) {
    const int taps_all = f.k_h * f.k_w;
    if (tile != nullptr && f.row_cx == 0 && f.sub_sh == 0 && f.flipped) {
        // Source [C][OC * taps]: 32 channels x 64 consecutive (oc, tap) entries per unit.
        const long long entries = static_cast<long long>(f.oc_n) * taps_all;
        const long long e_chunks = (entries + 63) / 64;
        const long long units = e_chunks * (f.cp / 32);
        for (long long u = block; u < units; u += blocks) {
            const int c0 = static_cast<int>(u / e_chunks) * 32;
            const long long e0 = (u % e_chunks) * 64;
            for (int i = threadIdx.x; i < 32 * 64; i += threads) {
                const int r = i >> 6, j = i & 63;
                const int ch = c0 + r;
                const long long e = e0 + j;
                tile[r * 65 + j] = (ch < f.c && e < entries) ? f.w[ch * entries + e] : 0.0f;
            }
            __syncthreads();
            for (int i = threadIdx.x; i < 32 * 64; i += threads) {
                const int j = i >> 5, r = i & 31;
                const long long e = e0 + j;
                if (e < entries) {
                    const long long oc = e / taps_all;
                    const int tap = static_cast<int>(e - oc * taps_all);
                    f.wp[(oc * taps_all + (taps_all - 1 - tap)) * f.cp + c0 + r] = tile[r * 65 + j];
                }
            }
            __syncthreads();
        }
        return;
    }
    if (tile != nullptr && f.row_cx == 0 && f.sub_sh == 0 && !f.flipped && taps_all <= 65) {
        // Source [OC][C * taps]: one output channel x `chunk` channels (all their taps) per unit.
        int chunk = (32 * 65 / taps_all) / 32 * 32;
        if (chunk > f.cp) chunk = f.cp;
        const int chunks = (f.cp + chunk - 1) / chunk;
        const long long units = static_cast<long long>(f.oc_n) * chunks;
        for (long long u = block; u < units; u += blocks) {
            const long long oc = u / chunks;
            const int c0 = static_cast<int>(u - oc * chunks) * chunk;
            const int real = min(chunk, f.c - c0);                     // channels that exist in w
            const float* src = f.w + (oc * f.c + c0) * taps_all;
            for (int i = threadIdx.x; i < real * taps_all; i += threads) tile[i] = src[i];
            __syncthreads();
            const int width = min(chunk, f.cp - c0);                   // channels written (zeros past C)
            float* dst = f.wp + oc * taps_all * f.cp + c0;
            for (int i = threadIdx.x; i < width * taps_all; i += threads) {
                const int tap = i / width, cc = i - tap * width;
                dst[static_cast<long long>(tap) * f.cp + cc] = cc < real ? tile[cc * taps_all + tap] : 0.0f;
            }
            __syncthreads();
        }
        return;
    }
    if (f.row_cx > 0) {
        const long long total = static_cast<long long>(f.oc_n) * f.k_h * UMMA_BK;
        for (long long i = block * threads + threadIdx.x; i < total; i += blocks * threads) {
            const int slot = static_cast<int>(i % UMMA_BK);
            const long long r = i / UMMA_BK;
            const int kh = static_cast<int>(r % f.k_h);
            const long long oc = r / f.k_h;
            const int kw = slot / f.row_cx, ch = slot - kw * f.row_cx;
            f.wp[i] = (kw < f.k_w && ch < f.c) ? f.w[((oc * f.c + ch) * f.k_h + kh) * f.k_w + kw] : 0.0f;
        }
        return;
    }
    const int taps = f.k_h * f.k_w;
    const long long total = static_cast<long long>(f.oc_n) * taps * f.cp;
    for (long long i = block * threads + threadIdx.x; i < total; i += blocks * threads) {
        const int ch = static_cast<int>(i % f.cp);
        const long long r = i / f.cp;
        const int tap = static_cast<int>(r % taps);
        const long long oc = r / taps;
        float v = 0.0f;
        if (ch < f.c) {
            if (f.flipped && f.sub_sh > 0) {
                const int kh = tap / f.k_w, kw = tap - kh * f.k_w;
                const int cls = static_cast<int>(oc / f.fwd_c), ci = static_cast<int>(oc - cls * f.fwd_c);
                const int a = cls / f.sub_sw, b = cls - a * f.sub_sw;
                const int j = f.pad_h - kh + f.lo_h[a], l = f.pad_w - kw + f.lo_w[b];
                const int fh = a + f.sub_sh * j, fw = b + f.sub_sw * l;
                if (j >= 0 && l >= 0 && fh < f.full_kh && fw < f.full_kw)
                    v = f.w[((static_cast<long long>(ch) * f.fwd_c + ci) * f.full_kh + fh) * f.full_kw + fw];
            } else if (f.flipped) {
                const int kh = tap / f.k_w, kw = tap - kh * f.k_w;
                v = f.w[((static_cast<long long>(ch) * f.oc_n + oc) * f.k_h + (f.k_h - 1 - kh)) * f.k_w +
                        (f.k_w - 1 - kw)];
            } else {
                v = f.w[(oc * f.c + ch) * taps + tap];
            }
        }
        f.wp[i] = v;
    }
}

// x[N][C][HW] -> xt[N][HW][Cx], Cx >= C (extra channels written as zero).
// 32-channel x 64-pixel tiles through shared memory: reads coalesce along HW, writes along C.
// With HW a multiple of 4 both sides move 128 bits per thread (a warp reads 512 contiguous
// bytes of one channel and writes four pixels' 128-byte channel runs); otherwise scalars.
// With `with_filters`, the blocks of the z slices past the batch pack the filters instead (one
// launch for both preparations of a convolution).
// With SCATTER, source pixel (r, q) of a src_w-wide plane lands at (r * d_h, q * d_w) of a
// dst_w-wide plane of dst_hw pixels per image (zeroed by the caller beforehand).
struct PixelScatter {
    int src_w, dst_w, dst_hw, d_h, d_w, first;      // `first`: destination pixel of source pixel 0
    __device__ __forceinline__ long long operator()(int p) const {
        const int r = p / src_w;
        return first + static_cast<long long>(r) * d_h * dst_w + static_cast<long long>(p - r * src_w) * d_w;
    }
};

template <bool VEC, bool SCATTER = false>
__global__ void __launch_bounds__(256)
nchw_to_nhwc_kernel(const float* __restrict__ x, float* __restrict__ xt, int c, int hw, int cx, int batch,
                    FilterPack filters, int with_filters, PixelScatter scatter = PixelScatter{}) {
    __shared__ float tile[32][65];
    // The tensor-core kernel that follows is launched with programmatic stream serialization: once every
    // block of this grid is running it may be set up (barriers, TMEM, descriptors) beside them; it waits
    // for this grid's completion itself before it loads anything.
    ptx::grid_launch_dependents();
    if (with_filters && int(blockIdx.z) >= batch) {
        const long long per_slice = static_cast<long long>(gridDim.x) * gridDim.y;
        pack_filters(filters, (int(blockIdx.z) - batch) * per_slice + blockIdx.y * gridDim.x + blockIdx.x,
                     per_slice * (int(gridDim.z) - batch), 256, &tile[0][0]);
        return;
    }
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 64;
    const int c0 = blockIdx.y * 32;
    const float* xn = x + static_cast<long long>(n) * c * hw;
    float* xtn = xt + static_cast<long long>(n) * (SCATTER ? scatter.dst_hw : hw) * cx;
    const int tid = threadIdx.x;
    if constexpr (VEC) {
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
            const int ch_l = pass * 16 + tid / 16, p_l = (tid % 16) * 4;
            const int ch = c0 + ch_l, p = p0 + p_l;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (ch < c && p < hw) v = *reinterpret_cast<const float4*>(xn + static_cast<long long>(ch) * hw + p);
            tile[ch_l][p_l + 0] = v.x;
            tile[ch_l][p_l + 1] = v.y;
            tile[ch_l][p_l + 2] = v.z;
            tile[ch_l][p_l + 3] = v.w;
        }
        __syncthreads();
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
            const int p_l = pass * 32 + tid / 8, ch_l = (tid % 8) * 4;
            const int p = p0 + p_l, ch = c0 + ch_l;
            if (p < hw && ch < cx)
                *reinterpret_cast<float4*>(xtn + (SCATTER ? scatter(p) : static_cast<long long>(p)) * cx + ch) =
                    make_float4(tile[ch_l][p_l], tile[ch_l + 1][p_l], tile[ch_l + 2][p_l], tile[ch_l + 3][p_l]);
        }
    } else {
        for (int i = tid; i < 32 * 64; i += 256) {
            const int ch_l = i / 64, p_l = i % 64;
            const int ch = c0 + ch_l, p = p0 + p_l;
            tile[ch_l][p_l] = (ch < c && p < hw) ? xn[static_cast<long long>(ch) * hw + p] : 0.0f;
        }
        __syncthreads();
        for (int i = tid; i < 32 * 64; i += 256) {
            const int p_l = i / 32, ch_l = i % 32;
            const int p = p0 + p_l, ch = c0 + ch_l;
            if (p < hw && ch < cx)
                xtn[(SCATTER ? scatter(p) : static_cast<long long>(p)) * cx + ch] = tile[ch_l][p_l];
        }
    }
}

// The same for at most four channels (cx == 4, a network's first layer), where the tiled kernel
// would leave most of its threads idle: a thread reads four consecutive pixels of every channel
// (128 bits each) and writes the four pixels' 16-byte channel groups.  hw must be a multiple of 4.
template <bool SCATTER>
__global__ void __launch_bounds__(256)
nchw_to_nhwc4_kernel(const float* __restrict__ x, float* __restrict__ xt, int c, int hw, int batch,
                     FilterPack filters, int with_filters, PixelScatter scatter) {
    ptx::grid_launch_dependents();      // see nchw_to_nhwc_kernel
    if (with_filters && int(blockIdx.z) >= batch) {
        const long long per_slice = static_cast<long long>(gridDim.x) * gridDim.y;
        pack_filters(filters, (int(blockIdx.z) - batch) * per_slice + blockIdx.y * gridDim.x + blockIdx.x,
                     per_slice * (int(gridDim.z) - batch), 256);
        return;
    }
    const int n = blockIdx.z;
    const int p = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (p >= hw) return;
    const float* xn = x + static_cast<long long>(n) * c * hw + p;
    float4 v[4];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch)
        v[ch] = ch < c ? *reinterpret_cast<const float4*>(xn + static_cast<long long>(ch) * hw)
                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4* dst = reinterpret_cast<float4*>(xt) + static_cast<long long>(n) * (SCATTER ? scatter.dst_hw : hw);
    dst[SCATTER ? scatter(p + 0) : p + 0] = make_float4(v[0].x, v[1].x, v[2].x, v[3].x);
    dst[SCATTER ? scatter(p + 1) : p + 1] = make_float4(v[0].y, v[1].y, v[2].y, v[3].y);
    dst[SCATTER ? scatter(p + 2) : p + 2] = make_float4(v[0].z, v[1].z, v[2].z, v[3].z);
    dst[SCATTER ? scatter(p + 3) : p + 3] = make_float4(v[0].w, v[1].w, v[2].w, v[3].w);
}

// ------------------------------------------------------------------ problem policy

template <int CTAS, bool ROW_PACKED = false, bool MULTI_IMAGE = false>
struct ConvProblem {
    // When a tile's pixels are contiguous in the output plane (box_w == OW) the output is the 2-D
    // tensor {OH*OW, N*OC} and goes out by bulk tensor stores like a GEMM's C; otherwise registers.
    static constexpr bool kTmaStore = true;
    // Few tiles and a long reduction (small feature maps, many channels): the K blocks of a tile
    // may be split over the CTA groups of a cluster.  Only the kernels for tiles of several images
    // carry that code: in the others it was never chosen for a layer that was measured, and its
    // presence alone costs the short tiles of large maps instruction-cache space.
    static constexpr bool kClusterSplit = MULTI_IMAGE;
    // Tiles of whole small planes may leave through compacted blocks (see has_plane_store).
    static constexpr bool kPlaneStore = MULTI_IMAGE;
    CUtensorMap map_w;     // packed filters: dims {KH*KW*Cp, OC}, box {32, 128}
    CUtensorMap map_x;     // NHWC input: dims {Cx, W, H, N}, box {32, box_w, box_h / CTAS, 1}
    CUtensorMap map_out;   // output planes: dims {OH*OW, N*OC}, box {32, 32}
    float* out;
    int oc_n, oh_n, ow_n;
    int box_w, box_h;      // output pixels per tile: box_h rows of box_w
    int box_n;             // MULTI_IMAGE: images per tile (each one whole: box_w >= OW, box_h >= OH)
    int tiles_w, tiles_h;  // tiles per image
    int c_blocks;          // Cp / 32
    int k_w;
    int p_h, p_w;
    int s_h, s_w;          // convolution strides: the box walks the input in these steps
    int total_kb;          // K blocks of the reduction: KH * KW * c_blocks
    int batch;
    // ROW_PACKED: one K block per filter row (see launch_conv), map_x is the window view.
    int contig;            // box_w == OW: the tile's pixels are contiguous in the output plane
    int vec_ok;            // 128-bit stores are aligned for every tile
    // Where output pixel (oh, ow) of plane (n, oc) goes: out + (n * OC + oc) * out_plane + out_off +
    // oh * out_row + ow * out_col.  A plain convolution has out_plane = OH * OW, out_off = 0,
    // out_row = OW, out_col = 1; a parity class of a strided grad_input writes every stride-th
    // pixel of a larger plane (then contig == 0).
    long long out_plane;
    int out_off, out_row, out_col;

    struct Tile {
        int oc0;           // first output channel of this CTA
        int n, oh0, ow0;   // image and first output pixel of the tile
        int hb0;           // first output row whose pixels this CTA stages as B
        int nb0;           // image whose pixels this CTA stages as B (MULTI_IMAGE: its first image)
    };

    __device__ __forceinline__ void prefetch_maps() const {
        ptx::prefetch_tensormap(&map_w);
        ptx::prefetch_tensormap(&map_x);
        ptx::prefetch_tensormap(&map_out);
    }
    __device__ __forceinline__ const CUtensorMap* out_map() const { return &map_out; }
    // Columns of a tile whose rows reach past OH map past the end of the plane and are clipped.
    // Rows past OC would land in the next image's planes: OC is a multiple of 32 on this path, so
    // a 32-row block is either whole or entirely past OC, and the latter is sent out of range.
    __device__ __forceinline__ void out_coords(const Tile& t, int row_in_cta, int c0, int& x, int& y) const {
        x = t.oh0 * ow_n + c0;
        y = t.n * oc_n + t.oc0 + row_in_cta;
        if (t.oc0 + row_in_cta >= oc_n) y = batch * oc_n;      // a block of rows past OC: clipped as a whole
    }
    __device__ __forceinline__ void finish(const Tile& t, int row_in_cta, int /*c0*/, float (&v)[32],
                                           const UmmaEpilogueArgs& epi) const {
        const int oc = t.oc0 + row_in_cta;
        if (epi.bias != nullptr && oc < oc_n) {
            const float b = __ldg(epi.bias + oc);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += b;
        }
        apply_activation(v, epi.act);
    }
    __device__ __forceinline__ Tile decode(int tm, int tn, uint32_t cta_rank) const {
        Tile t;
        t.oc0 = (tm * CTAS + int(cta_rank)) * UMMA_BM;
        if constexpr (MULTI_IMAGE) {
            // The CTAs of a pair split the tile's images, not its rows, so the accumulator
            // columns stay in (image, row, column) order.
            t.n = tn * box_n;
            t.oh0 = t.ow0 = t.hb0 = 0;
            t.nb0 = t.n + int(cta_rank) * (box_n / CTAS);
            return t;
        }
        const int per_image = tiles_h * tiles_w;
        t.n = tn / per_image;
        const int r = tn - t.n * per_image;
        const int th = r / tiles_w;
        t.oh0 = th * box_h;
        t.ow0 = (r - th * tiles_w) * box_w;
        t.hb0 = t.oh0 + int(cta_rank) * (box_h / CTAS);
        t.nb0 = t.n;
        return t;
    }
    __device__ __forceinline__ int plane_columns() const { return box_w * box_h; }
    __device__ __forceinline__ uint32_t plane_bytes() const { return 32u * uint32_t(oh_n * ow_n) * 4u; }
    __device__ __forceinline__ float* plane_dst(const Tile& t, int row0, int plane) const {
        const int oc = t.oc0 + row0;
        if (oc >= oc_n || t.n + plane >= batch) return nullptr;     // OC is a multiple of 32 in this mode
        return out + (static_cast<long long>(t.n + plane) * oc_n + oc) * out_plane;
    }
    // Row `lane` of the block is that output channel's plane, OH * OW floats; columns of the pixel
    // box past OW or OH are dropped.  (An odd plane size keeps the lanes on different banks.)
    __device__ __forceinline__ void plane_stage(uint32_t staging, uint32_t lane, int col_in_plane,
                                                const float (&v)[32]) const {
        const uint32_t row = staging + lane * uint32_t(oh_n * ow_n) * 4u;
        int oh = col_in_plane / box_w;
        int ow = col_in_plane - oh * box_w;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (oh < oh_n && ow < ow_n) ptx::st_shared_f32(row + uint32_t(oh * ow_n + ow) * 4u, v[j]);
            if (++ow == box_w) { ow = 0; ++oh; }
        }
    }
    template <int C>
    __device__ __forceinline__ void load(const Tile& t, int kb, uint32_t a_smem, uint32_t b_smem,
                                         uint32_t bar) const {
        const int tap = kb / c_blocks;
        const int c0 = (kb - tap * c_blocks) * UMMA_BK;
        // Row-packed: K block kb is filter row kb, and coordinate 1 counts output columns (each
        // the start of a window of KW pixels in the width-padded copy).
        const int kh = ROW_PACKED ? kb : tap / k_w;
        const int x1 = ROW_PACKED ? t.ow0 : t.ow0 * s_w + (tap - kh * k_w) - p_w;
        // A K block past the end of the reduction (a stage's padding) must read zeros on
        // both sides: the filter coordinate is out of range by itself, the image index is
        // pushed out of range here.
        const int n = kb < total_kb ? t.nb0 : batch;
        if constexpr (C == 1) {
            ptx::tma_load_2d(a_smem, &map_w, bar, kb * UMMA_BK, t.oc0);
            ptx::tma_load_4d(b_smem, &map_x, bar, c0, x1, t.hb0 * s_h + kh - p_h, n);
        } else {
            ptx::tma_load_2d_pair(a_smem, &map_w, bar, kb * UMMA_BK, t.oc0);
            ptx::tma_load_4d_pair(b_smem, &map_x, bar, c0, x1, t.hb0 * s_h + kh - p_h, n);
        }
    }
    __device__ __forceinline__ void store(const Tile& t, int row_in_cta, int c0, float (&v)[32],
                                          const UmmaEpilogueArgs& epi, int /*mode: tiles are never split*/) const {
        const int oc = t.oc0 + row_in_cta;
        if (oc >= oc_n) return;
        if (epi.bias != nullptr) {
            const float b = __ldg(epi.bias + oc);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += b;
        }
        apply_activation(v, epi.act);
        if constexpr (MULTI_IMAGE) {
            const int per_image = box_w * box_h;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int col = c0 + j;
                const int img = col / per_image;
                const int rem = col - img * per_image;
                const int oh = rem / box_w, ow = rem - oh * box_w;
                if (t.n + img < batch && oh < oh_n && ow < ow_n)
                    out[(static_cast<long long>(t.n + img) * oc_n + oc) * out_plane + out_off + oh * out_row +
                        ow * out_col] = v[j];
            }
            return;
        }
        float* plane = out + (static_cast<long long>(t.n) * oc_n + oc) * out_plane + out_off;
        if (contig) {
            const int rows = min(box_h, oh_n - t.oh0);
            const int limit = rows * ow_n;                 // valid accumulator columns
            float* dst = plane + static_cast<long long>(t.oh0) * ow_n + c0;
            if (vec_ok && c0 + 32 <= limit) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (c0 + j < limit) dst[j] = v[j];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int col = c0 + j;
                const int r = col / box_w;
                const int q = col - r * box_w;
                const int oh = t.oh0 + r, ow = t.ow0 + q;
                if (oh < oh_n && ow < ow_n) plane[static_cast<long long>(oh) * out_row + ow * out_col] = v[j];
            }
        }
    }
};

// Stride-1 convolutions with three taps per filter row over whole output rows: the form
// umma_gemm.cuh describes under has_shared_b.  A stage is one filter row kh and one block of 32
// channels: three filter slabs (kw = 0, 1, 2) and the input pixels under them - `rows_per_half`
// image rows per CTA, OW + 2 pixels each, halo included - loaded once and read by the three taps at
// offsets of 0, 1 and 2 pixels.  Operand column n of a CTA's share is pixel (n / pitch, n % pitch) of
// its rows; the columns with n % pitch >= OW (and those past rows_per_half * pitch) are by-products.
// CTAS = 2: the CTAs of a pair stage half of the tile's rows each; CTAS = 1 (at most 128 output
// channels): one CTA stages them all.
template <int CTAS>
struct ConvRowProblem {
    static constexpr bool kTmaStore = true;
    static constexpr bool kClusterSplit = false;
    static constexpr bool kSharedB = true;
    CUtensorMap map_w;     // packed filters: dims {KH*3*Cp, OC}, box {32, 128}
    CUtensorMap map_x;     // NHWC input: dims {Cx, W, H, N}, box {32, pitch, rows_per_half, 1}
    CUtensorMap map_out;   // output: dims {OW, OH, N*OC}, box {OW, 1, 32}, not swizzled
    int oc_n, oh_n, ow_n, batch;
    int rows_per_half, pitch, half_cols;
    int tiles_h;           // tiles per image
    int c_blocks, cp, p_h, p_w;

    struct Tile {
        int oc0, n, oh0, hb0;
    };
    __device__ __forceinline__ void prefetch_maps() const {
        ptx::prefetch_tensormap(&map_w);
        ptx::prefetch_tensormap(&map_x);
        ptx::prefetch_tensormap(&map_out);
    }
    __device__ __forceinline__ const CUtensorMap* out_map() const { return &map_out; }
    __device__ __forceinline__ Tile decode(int tm, int tn, uint32_t cta_rank) const {
        Tile t;
        t.oc0 = (tm * CTAS + int(cta_rank)) * UMMA_BM;
        t.n = tn / tiles_h;
        t.oh0 = (tn - t.n * tiles_h) * (CTAS * rows_per_half);
        t.hb0 = t.oh0 + int(cta_rank) * rows_per_half;
        return t;
    }
    template <int C>
    __device__ __forceinline__ void load_stage(const Tile& t, int stage_index, uint32_t a_smem, uint32_t b_smem,
                                               uint32_t bar) const {
        static_assert(C == CTAS, "loads follow the CTA grouping of the problem");
        const int kh = stage_index / c_blocks;
        const int c0 = (stage_index - kh * c_blocks) * UMMA_BK;
#pragma unroll
        for (int kw = 0; kw < 3; ++kw) {
            const uint32_t dst = a_smem + kw * (UMMA_BM * UMMA_BK * 4);
            if constexpr (C == 2) ptx::tma_load_2d_pair(dst, &map_w, bar, (kh * 3 + kw) * cp + c0, t.oc0);
            else ptx::tma_load_2d(dst, &map_w, bar, (kh * 3 + kw) * cp + c0, t.oc0);
        }
        if constexpr (C == 2) ptx::tma_load_4d_pair(b_smem, &map_x, bar, c0, -p_w, t.hb0 + kh - p_h, t.n);
        else ptx::tma_load_4d(b_smem, &map_x, bar, c0, -p_w, t.hb0 + kh - p_h, t.n);
    }
    __device__ __forceinline__ void finish(const Tile& t, int row_in_cta, int /*c0*/, float (&v)[32],
                                           const UmmaEpilogueArgs& epi) const {
        const int oc = t.oc0 + row_in_cta;
        if (epi.bias != nullptr && oc < oc_n) {
            const float b = __ldg(epi.bias + oc);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += b;
        }
        apply_activation(v, epi.act);
    }
    __device__ __forceinline__ int out_rows() const { return CTAS * rows_per_half; }
    __device__ __forceinline__ int row_values() const { return ow_n; }
    __device__ __forceinline__ uint32_t row_column(int r) const {
        const int half = r / rows_per_half;
        return uint32_t(half * half_cols + (r - half * rows_per_half) * pitch);
    }
    // Rows past OH and blocks of channels past OC (a multiple of 32) are clipped by the store.
    __device__ __forceinline__ void row_coords(const Tile& t, int row0, int r, int& x, int& y, int& z) const {
        x = 0;
        y = t.oh0 + r;
        z = t.n * oc_n + t.oc0 + row0;
        if (t.oc0 + row0 >= oc_n) z = batch * oc_n;
    }
    // Never used: every tile leaves through the row stores.
    __device__ __forceinline__ void store(const Tile&, int, int, float (&)[32], const UmmaEpilogueArgs&, int) const {}
    __device__ __forceinline__ void out_coords(const Tile&, int, int, int& x, int& y) const { x = y = 0; }
};

// The same sharing for small feature maps (7 x 7 and the like) on CTA pairs: a tile is four whole images,
// two per CTA; a stage holds the three filter slabs of (kh, 32 channels) and, per image, the OH input
// rows under filter row kh with OW + 2 pixels each (at most 63 pixels, in a slot of 64 operand rows).
// Operand column n of an image is pixel (n / pitch, n % pitch).  The reduction may be split over the
// pairs of a cluster, and the tile leaves as compacted planes (has_plane_store), both as for ConvProblem.
struct ConvSmallMapProblem {
    static constexpr bool kTmaStore = true;        // (finish() is used; no output map: tma_store stays 0)
    static constexpr bool kClusterSplit = true;
    static constexpr bool kSharedB = true;
    static constexpr bool kPlaneStore = true;
    CUtensorMap map_w;     // packed filters: dims {KH*3*Cp, OC}, box {32, 128}
    CUtensorMap map_x;     // NHWC input: dims {Cx, W, H, N}, box {32, pitch, OH, 1}
    float* out;
    int oc_n, oh_n, ow_n, batch;
    int pitch;             // OW + 2
    int c_blocks, cp, p_h, p_w;
    int total_stages;      // KH * c_blocks

    struct Tile {
        int oc0, n, nb0;
    };
    __device__ __forceinline__ void prefetch_maps() const {
        ptx::prefetch_tensormap(&map_w);
        ptx::prefetch_tensormap(&map_x);
    }
    __device__ __forceinline__ const CUtensorMap* out_map() const { return &map_w; }      // never used
    __device__ __forceinline__ void out_coords(const Tile&, int, int, int& x, int& y) const { x = y = 0; }
    __device__ __forceinline__ Tile decode(int tm, int tn, uint32_t cta_rank) const {
        Tile t;
        t.oc0 = (tm * 2 + int(cta_rank)) * UMMA_BM;
        t.n = tn * 4;
        t.nb0 = t.n + int(cta_rank) * 2;
        return t;
    }
    template <int C>
    __device__ __forceinline__ void load_stage(const Tile& t, int stage_index, uint32_t a_smem, uint32_t b_smem,
                                               uint32_t bar) const {
        static_assert(C == 2, "small maps run on CTA pairs");
        const int kh = stage_index / c_blocks;
        const int c0 = (stage_index - kh * c_blocks) * UMMA_BK;
        // A stage past the end of a K range that is not a whole number of stages cannot occur: the
        // ranges are counted in stages.
#pragma unroll
        for (int kw = 0; kw < 3; ++kw)
            ptx::tma_load_2d_pair(a_smem + kw * (UMMA_BM * UMMA_BK * 4), &map_w, bar, (kh * 3 + kw) * cp + c0, t.oc0);
#pragma unroll
        for (int i = 0; i < 2; ++i)      // an image past the batch reads zeros
            ptx::tma_load_4d_pair(b_smem + i * (64 * 128), &map_x, bar, c0, -p_w, kh - p_h, t.nb0 + i);
    }
    __device__ __forceinline__ void finish(const Tile& t, int row_in_cta, int /*c0*/, float (&v)[32],
                                           const UmmaEpilogueArgs& epi) const {
        const int oc = t.oc0 + row_in_cta;
        if (epi.bias != nullptr && oc < oc_n) {
            const float b = __ldg(epi.bias + oc);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += b;
        }
        apply_activation(v, epi.act);
    }
    __device__ __forceinline__ int plane_columns() const { return 64; }
    __device__ __forceinline__ uint32_t plane_bytes() const { return 32u * uint32_t(oh_n * ow_n) * 4u; }
    __device__ __forceinline__ float* plane_dst(const Tile& t, int row0, int plane) const {
        const int oc = t.oc0 + row0;
        if (oc >= oc_n || t.n + plane >= batch) return nullptr;
        return out + (static_cast<long long>(t.n + plane) * oc_n + oc) * (oh_n * ow_n);
    }
    __device__ __forceinline__ void plane_stage(uint32_t staging, uint32_t lane, int col_in_plane,
                                                const float (&v)[32]) const {
        const uint32_t row = staging + lane * uint32_t(oh_n * ow_n) * 4u;
        int oh = col_in_plane / pitch;
        int ow = col_in_plane - oh * pitch;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (oh < oh_n && ow < ow_n) ptx::st_shared_f32(row + uint32_t(oh * ow_n + ow) * 4u, v[j]);
            if (++ow == pitch) { ow = 0; ++oh; }
        }
    }
    // Never used: every tile leaves as compacted planes.
    __device__ __forceinline__ void store(const Tile&, int, int, float (&)[32], const UmmaEpilogueArgs&, int) const {}
};

// Whether that form takes a convolution: CTA pairs, three taps per filter row, stride 1, an image's
// OH x (OW + 2) operand columns within 64, planes the compacted stores take (an odd number of floats,
// at most 64), output the same size as the input (so the OH rows under filter row kh are one box).
bool small_map_form_applies(const ConvShape& s, int ctas, const float* out, bool plain_output) {
    const int oh = s.out_h(), ow = s.out_w();
    if (ctas != 2 || !plain_output || s.k_w != 3 || s.s_h != 1 || s.s_w != 1 || s.batch < 4) return false;
    if (oh * (ow + 2) > 64 || ow + 2 > 16 || (oh * ow) % 2 == 0 || oh * ow > 64) return false;
    return s.out_c % 32 == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
}

void launch_conv_small_maps(const float* xt, const float* wp, const float* bias, float* out, const ConvShape& s,
                            int cx, int cp, int act, cudaStream_t stream) {
    constexpr int KW = 3;
    using Cfg = UmmaConfig<2, 256, false, KW>;
    const DeviceInfo& dev = device_info();
    const int oh = s.out_h(), ow = s.out_w();
    ConvSmallMapProblem prob;
    {
        const uint64_t dims[2] = {uint64_t(s.k_h) * KW * cp, uint64_t(s.out_c)};
        const uint64_t strides[1] = {uint64_t(s.k_h) * KW * cp * 4};
        const uint32_t box[2] = {UMMA_BK, UMMA_BM};
        encode_tensor_map(&prob.map_w, wp, 2, dims, strides, box, TmaSwizzle::B128);
    }
    {
        const uint64_t dims[4] = {uint64_t(cx), uint64_t(s.in_w), uint64_t(s.in_h), uint64_t(s.batch)};
        const uint64_t strides[3] = {uint64_t(cx) * 4, uint64_t(s.in_w) * cx * 4, uint64_t(s.in_h) * s.in_w * cx * 4};
        const uint32_t box[4] = {UMMA_BK, uint32_t(ow + 2), uint32_t(oh), 1};
        encode_tensor_map(&prob.map_x, xt, 4, dims, strides, box, TmaSwizzle::B128);
    }
    prob.out = out;
    prob.oc_n = s.out_c;
    prob.oh_n = oh;
    prob.ow_n = ow;
    prob.batch = s.batch;
    prob.pitch = ow + 2;
    prob.c_blocks = cp / UMMA_BK;
    prob.cp = cp;
    prob.p_h = s.p_h;
    prob.p_w = s.p_w;
    prob.total_stages = s.k_h * prob.c_blocks;

    constexpr uint32_t stage_bytes = KW * Cfg::A_BYTES + Cfg::B_BYTES;
    const uint32_t tx = 2u * (KW * Cfg::A_BYTES + 2u * uint32_t(ow + 2) * oh * UMMA_BK * 4);
    UmmaSchedule sched = whole_tile_schedule((s.out_c + 2 * UMMA_BM - 1) / (2 * UMMA_BM), (s.batch + 3) / 4,
                                             prob.total_stages, 256, tx, 8, dev.status_word);
    sched.raster_group = sched.tiles_m;
    sched.plane_store = 1;
    const long long num_tiles = static_cast<long long>(sched.tiles_m) * sched.tiles_n;
    // Two K ranges per tile, on the two pairs of a cluster, when every tile finds its cluster at once
    // and a range still has a few stages.
    int ksplit = 1;
    if (num_tiles * 4 <= dev.num_sms * 7 / 8 && prob.total_stages >= 8 && prob.total_stages % 2 == 0) ksplit = 2;
    uint32_t exchange_bytes = 0, staging_bytes = UMMA_STORE_STAGING_BYTES;
    if (ksplit > 1) {
        sched.cluster_split = ksplit;
        sched.kb_per_split = prob.total_stages / ksplit;
        exchange_bytes = uint32_t(ksplit - 1) * UMMA_BM * uint32_t(256 / ksplit) * 4u;
        staging_bytes = 0;                         // split tiles stage in the idle stage ring
    }
    sched.exchange_bytes = exchange_bytes;
    sched.stages = int((Cfg::SMEM_BUDGET - exchange_bytes - staging_bytes) / stage_bytes);
    const uint32_t smem_bytes = uint32_t(sched.stages) * stage_bytes + exchange_bytes + staging_bytes + 1024;
    long long groups = dev.num_sms / 2;
    if (groups > num_tiles) groups = num_tiles;
    if (ksplit > 1) groups = num_tiles;
    CB200_TRACE("conv2d implicit GEMM tcgen05, small maps with rows shared by the taps of a filter row: N=%d C=%d "
                "%dx%d -> OC=%d %dx%d, %dx3 pad %dx%d; four images of %d x %d pixels per tile, stages=%d of %u KB, "
                "clusters=%lld, stages per tile=%d, cluster_split=%d, store=bulk planes",
                s.batch, s.in_c, s.in_h, s.in_w, s.out_c, oh, ow, s.k_h, s.p_h, s.p_w, oh, ow + 2, sched.stages,
                stage_bytes / 1024, groups, sched.k_blocks, ksplit);
    auto kernel = umma_tf32_kernel<2, 256, false, KW, ConvSmallMapProblem>;
    UmmaEpilogueArgs epi{bias, 1, act};
    launch_umma(kernel, prob, sched, epi, groups, 2 * ksplit, smem_bytes, Cfg::SMEM_MAX, stream);
}

struct RowPlan {
    int rows_per_half = 0, pitch = 0, half_cols = 0;
};

// Whether (and how) the row form takes a convolution: three taps per filter row, stride 1, whole output
// rows of 16-byte multiples; a CTA's share of the operand columns is at most 120 in a pair and 248 alone.
RowPlan plan_rows(const ConvShape& s, int ctas, const float* out, bool plain_output) {
    RowPlan p;
    const int oh = s.out_h(), ow = s.out_w();
    if (!plain_output || s.k_w != 3 || s.s_h != 1 || s.s_w != 1) return p;
    if (ow % 4 != 0 || ow < 24 || ow > 64 || s.out_c % 32 != 0 || (reinterpret_cast<uintptr_t>(out) & 15u) != 0) return p;
    const int pitch = ow + 2;
    const int share = ctas == 2 ? 120 : 248;
    int rows = share / pitch;
    const int rows_needed = (oh + ctas - 1) / ctas;
    if (rows > rows_needed) rows = rows_needed;
    if (rows < 1) return p;
    // A pair's MMA has N = 2 x share (a multiple of 16), a single CTA's N = share (likewise).
    const int half_cols = round_up_int(rows * pitch, ctas == 2 ? 8 : 16);
    // The epilogue reads 32 or 64 accumulator columns from the start of a row: inside the buffer.
    const int last_row = (ctas - 1) * half_cols + (rows - 1) * pitch;
    if (last_row + (ow > 32 ? 64 : 32) > 256) return p;
    p.rows_per_half = rows;
    p.pitch = pitch;
    p.half_cols = half_cols;
    return p;
}

template <int CTAS>
void launch_conv_rows(const float* xt, const float* wp, const float* bias, float* out, const ConvShape& s, int cx,
                      int cp, const RowPlan& plan, int act, cudaStream_t stream) {
    constexpr int KW = 3;
    using Cfg = UmmaConfig<CTAS, 256, false, KW>;
    const DeviceInfo& dev = device_info();
    const int oh = s.out_h(), ow = s.out_w();
    ConvRowProblem<CTAS> prob;
    {
        const uint64_t dims[2] = {uint64_t(s.k_h) * KW * cp, uint64_t(s.out_c)};
        const uint64_t strides[1] = {uint64_t(s.k_h) * KW * cp * 4};
        const uint32_t box[2] = {UMMA_BK, UMMA_BM};
        encode_tensor_map(&prob.map_w, wp, 2, dims, strides, box, TmaSwizzle::B128);
    }
    {
        const uint64_t dims[4] = {uint64_t(cx), uint64_t(s.in_w), uint64_t(s.in_h), uint64_t(s.batch)};
        const uint64_t strides[3] = {uint64_t(cx) * 4, uint64_t(s.in_w) * cx * 4, uint64_t(s.in_h) * s.in_w * cx * 4};
        const uint32_t box[4] = {UMMA_BK, uint32_t(plan.pitch), uint32_t(plan.rows_per_half), 1};
        encode_tensor_map(&prob.map_x, xt, 4, dims, strides, box, TmaSwizzle::B128);
    }
    {
        const uint64_t dims[3] = {uint64_t(ow), uint64_t(oh), uint64_t(s.batch) * s.out_c};
        const uint64_t strides[2] = {uint64_t(ow) * 4, uint64_t(oh) * ow * 4};
        const uint32_t box[3] = {uint32_t(ow), 1, 32};
        encode_tensor_map(&prob.map_out, out, 3, dims, strides, box, TmaSwizzle::None);
    }
    prob.oc_n = s.out_c;
    prob.oh_n = oh;
    prob.ow_n = ow;
    prob.batch = s.batch;
    prob.rows_per_half = plan.rows_per_half;
    prob.pitch = plan.pitch;
    prob.half_cols = plan.half_cols;
    prob.tiles_h = (oh + CTAS * plan.rows_per_half - 1) / (CTAS * plan.rows_per_half);
    prob.c_blocks = cp / UMMA_BK;
    prob.cp = cp;
    prob.p_h = s.p_h;
    prob.p_w = s.p_w;

    constexpr uint32_t stage_bytes = KW * Cfg::A_BYTES + Cfg::B_BYTES;
    const int umma_n = CTAS * plan.half_cols;
    const uint32_t tx = uint32_t(CTAS) * (KW * Cfg::A_BYTES + uint32_t(plan.pitch) * plan.rows_per_half * UMMA_BK * 4);
    const int stages = int((Cfg::SMEM_BUDGET - UMMA_STORE_STAGING_BYTES) / stage_bytes);
    UmmaSchedule sched = whole_tile_schedule((s.out_c + CTAS * UMMA_BM - 1) / (CTAS * UMMA_BM), s.batch * prob.tiles_h,
                                             s.k_h * prob.c_blocks, umma_n, tx, stages, dev.status_word);
    sched.raster_group = sched.tiles_m;
    const uint32_t smem_bytes = uint32_t(stages) * stage_bytes + UMMA_STORE_STAGING_BYTES + 1024;
    const long long num_tiles = static_cast<long long>(sched.tiles_m) * sched.tiles_n;
    CB200_REQUIRE(num_tiles < (1LL << 30), "conv2d: too many tiles");
    long long groups = dev.num_sms / CTAS;
    if (groups > num_tiles) groups = num_tiles;
    CB200_TRACE("conv2d implicit GEMM tcgen05, rows shared by the taps of a filter row: N=%d C=%d %dx%d -> OC=%d "
                "%dx%d, %dx3 pad %dx%d; %d rows x %d pixels per CTA = %d columns per MMA, ctas/mma=%d, stages=%d of %u KB, "
                "clusters=%lld, stages per tile=%d",
                s.batch, s.in_c, s.in_h, s.in_w, s.out_c, oh, ow, s.k_h, s.p_h, s.p_w, plan.rows_per_half, plan.pitch,
                umma_n, CTAS, stages, stage_bytes / 1024, groups, sched.k_blocks);
    auto kernel = umma_tf32_kernel<CTAS, 256, false, KW, ConvRowProblem<CTAS>>;
    UmmaEpilogueArgs epi{bias, 1, act};
    launch_umma(kernel, prob, sched, epi, groups, CTAS, smem_bytes, Cfg::SMEM_MAX, stream);
}

struct TilePlan {
    int box_w = 0, box_h = 0;
    int box_n = 1;      // > 1: whole images per tile (small feature maps)
    int ksplit = 1;     // > 1: the reduction is split over this many CTA groups of one cluster
};

// Output-pixel box of one tile: box_h rows of box_w pixels, box_w * box_h a
// multiple of 32 and at most 256, box_h a multiple of the CTAs that split it;
// picked to waste the fewest accumulator columns, then to be as large as possible.
// With strides the TMA box spans box * stride input pixels, which must stay within 256 per dimension.
TilePlan plan_tile(int oh, int ow, int ctas, int s_h, int s_w) {
    TilePlan best;
    double best_eff = -1.0;
    const int max_w = 256 / s_w, max_h = 256 / s_h * ctas;
    const int w_lo = ow < max_w ? ow : max_w;
    const int w_hi = (w_lo + 31 < max_w) ? w_lo + 31 : max_w;
    for (int bw = w_lo; bw <= w_hi; ++bw) {
        for (int bh = ctas; bh * bw <= 256; bh += ctas) {
            if ((bh * bw) % 32 != 0) continue;
            if (bh > max_h || bw > max_w) continue;
            const int tiles_w = (ow + bw - 1) / bw;
            const int tiles_h = (oh + bh - 1) / bh;
            const double eff = double(oh) * ow / (double(tiles_w) * tiles_h * bw * bh);
            const double score = eff + 1e-4 * (bw * bh) / 256.0;
            if (score > best_eff) {
                best_eff = score;
                best.box_w = bw;
                best.box_h = bh;
            }
        }
    }
    return best;
}

// Small feature maps: a tile of box_n whole images (box_w >= OW, box_h >= OH, box_n a multiple of
// the CTAs that split it), so that the filter slab a CTA stages per K block is used by more
// accumulator columns than one image's 49 or 16.  And few tiles with a long reduction: the K blocks
// of a tile split over `ksplit` CTA groups of one cluster, which add their partial sums through
// distributed shared memory (one tile per cluster, so every tile must find a cluster in one wave
// for the split to pay).  Candidates are ranked by an estimate of the launch's K loop: per K block
// the slower of the tensor pipe (about 1.08 ns per accumulator column) and the CTA's operand ingest
// (about 114 bytes per ns), times the K blocks of a group, times the waves of tiles over the SMs,
// plus what the exchange of partial sums costs.  Few large tiles leave SMs idle, many small ones
// re-read the filters.
constexpr double kExchangeNs = 3500.0, kExchangeDoublingNs = 750.0;

// Whether `ksplit` groups of `ctas` CTAs can share a tile of n accumulator columns: a portable
// cluster, whole 32-column chunks per group, and room for the exchange buffer beside two stages.
bool cluster_split_fits(int n, int ctas, int ksplit, int k_blocks, int katoms) {
    if (ksplit == 1) return true;
    if (ctas * ksplit > 8 || n % (32 * ksplit) != 0) return false;
    int per = (k_blocks + ksplit - 1) / ksplit;
    per = (per + katoms - 1) / katoms * katoms;
    if (per < 2 * katoms || (k_blocks + per - 1) / per != ksplit) return false;
    const uint32_t stage = uint32_t(katoms) * (UMMA_BM * UMMA_BK * 4 + uint32_t(n / ctas) * UMMA_BK * 4);
    const uint32_t exchange = uint32_t(ksplit - 1) * UMMA_BM * uint32_t(n / ksplit) * 4u;
    // (A split tile stages its stores in the idle stage ring, which two stages always cover.)
    return exchange + 2 * stage <= 232448u - 1536u;     // the kernels' shared-memory budget
}

TilePlan plan_multi_image_tile(int oh, int ow, int batch, int ctas, int s_h, int s_w, int tiles_m, int num_sms,
                               int k_blocks, const TilePlan& single) {
    TilePlan best = single;
    const int katoms = ctas == 2 ? 2 : 1;
    auto cost_of = [&](int bw, int bh, int bn, long long pixel_tiles, int ksplit) {
        const int n = bw * bh * bn;
        const double mma_ns = 1.08 * n;
        const double ingest_ns = (UMMA_BM * UMMA_BK * 4 + double(n / ctas) * UMMA_BK * 4) / 114.0;
        const int slots = num_sms / (ctas * ksplit) > 0 ? num_sms / (ctas * ksplit) : 1;
        const long long tiles = pixel_tiles * tiles_m;
        const long long waves = (tiles + slots - 1) / slots;
        double exchange_ns = 0.0;
        if (ksplit > 1) {
            if (waves > 1) return 1e30;
            exchange_ns = kExchangeNs;
            for (int k = ksplit; k > 2; k /= 2) exchange_ns += kExchangeDoublingNs;
        }
        const int per = (k_blocks + ksplit - 1) / ksplit;
        return double(waves) * per * (mma_ns > ingest_ns ? mma_ns : ingest_ns) + exchange_ns;
    };
    double best_cost = 1e30;
    if (single.box_w > 0) {
        const long long tiles = static_cast<long long>((ow + single.box_w - 1) / single.box_w) *
                                ((oh + single.box_h - 1) / single.box_h) * batch;
        best_cost = cost_of(single.box_w, single.box_h, 1, tiles, 1);
    }
    if (oh * ow > 128 || batch < 2) return best;
    for (int bw = ow; bw <= ow + 7 && bw * s_w <= 256; ++bw)
        for (int bh = oh; bh <= oh + 7 && bh * s_h <= 256; ++bh)
            for (int bn = ctas; bw * bh * bn <= 256; bn += ctas) {
                if (bn < 2 || (bw * bh * bn) % 32 != 0) continue;
                for (int ks = 1; ks <= 4; ks *= 2) {
                    if (!cluster_split_fits(bw * bh * bn, ctas, ks, k_blocks, katoms)) continue;
                    const double cost = cost_of(bw, bh, bn, (batch + bn - 1) / bn, ks);
                    if (cost < best_cost * 0.999) {
                        best_cost = cost;
                        best.box_w = bw;
                        best.box_h = bh;
                        best.box_n = bn;
                        best.ksplit = ks;
                    }
                }
            }
    return best;
}

// What a parity class of a strided grad_input changes about a launch: the input plane the tensor
// map describes (rows and columns past it read as zeros, and `s` may claim a larger or smaller
// plane so that its output size is the class's), and where the output pixels go.
struct ConvExtras {
    int map_h, map_w;                 // true extent of the input plane
    long long out_plane;              // floats per output plane
    int out_off, out_row, out_col;    // see ConvProblem
    bool scattered;                   // the output pixels are not a dense OH x OW plane
};

template <int CTAS, int KATOMS, bool ROW_PACKED, bool MULTI_IMAGE>
void launch_conv(const float* xt, const float* wp, const float* bias, float* out, const ConvShape& s,
                 int cx, int cp, const TilePlan& plan, int act, cudaStream_t stream,
                 const ConvExtras* extras = nullptr) {
    using Cfg = UmmaConfig<CTAS, 256, false, KATOMS>;
    using Prob = ConvProblem<CTAS, ROW_PACKED, MULTI_IMAGE>;
    // Rows and images of the pixel box one CTA stages.
    const uint32_t cta_rows = uint32_t(MULTI_IMAGE ? plan.box_h : plan.box_h / CTAS);
    const uint32_t cta_images = uint32_t(MULTI_IMAGE ? plan.box_n / CTAS : 1);
    constexpr bool row_packed = ROW_PACKED;
    const DeviceInfo& dev = device_info();
    const int oh = s.out_h(), ow = s.out_w();
    // Row-packed: the K blocks are the KH filter rows, each one 32-wide block.
    const int taps = row_packed ? s.k_h : s.k_h * s.k_w;

    Prob prob;
    {
        const uint64_t dims[2] = {uint64_t(taps) * cp, uint64_t(s.out_c)};
        const uint64_t strides[1] = {uint64_t(taps) * cp * 4};
        const uint32_t box[2] = {UMMA_BK, UMMA_BM};
        encode_tensor_map(&prob.map_w, wp, 2, dims, strides, box, TmaSwizzle::B128);
    }
    if (row_packed) {
        // The input copy is [N][H][W + 2 * pad_w][cx] with the padding columns zero.  Seen as
        // {KW * cx, OW, H, N} with a step of stride_w pixels between output columns, row (q, h, n)
        // is the window of KW pixels x cx channels that output column q reads from input row h:
        // contiguous in memory, overlapping its neighbours'.  A 32-wide box reads zeros past KW * cx.
        const int wp_pixels = s.in_w + 2 * s.p_w;
        const uint64_t dims[4] = {uint64_t(s.k_w) * cx, uint64_t(ow), uint64_t(s.in_h), uint64_t(s.batch)};
        const uint64_t strides[3] = {uint64_t(s.s_w) * cx * 4, uint64_t(wp_pixels) * cx * 4,
                                     uint64_t(s.in_h) * wp_pixels * cx * 4};
        const uint32_t box[4] = {UMMA_BK, uint32_t(plan.box_w), cta_rows * s.s_h, cta_images};
        const uint32_t steps[4] = {1, 1, uint32_t(s.s_h), 1};
        encode_tensor_map(&prob.map_x, xt, 4, dims, strides, box, TmaSwizzle::B128, steps);
    } else {
        const int map_h = extras ? extras->map_h : s.in_h, map_w = extras ? extras->map_w : s.in_w;
        const uint64_t dims[4] = {uint64_t(cx), uint64_t(map_w), uint64_t(map_h), uint64_t(s.batch)};
        const uint64_t strides[3] = {uint64_t(cx) * 4, uint64_t(map_w) * cx * 4,
                                     uint64_t(map_h) * map_w * cx * 4};
        // A strided convolution reads every s-th input pixel: the box spans box * s input pixels
        // and the TMA unit walks it in steps of s (element strides), so box_w x box_h pixels land.
        const uint32_t box[4] = {UMMA_BK, uint32_t(plan.box_w * s.s_w), cta_rows * s.s_h, cta_images};
        const uint32_t steps[4] = {1, uint32_t(s.s_w), uint32_t(s.s_h), 1};
        encode_tensor_map(&prob.map_x, xt, 4, dims, strides, box, TmaSwizzle::B128, steps);
    }
    prob.out = out;
    prob.oc_n = s.out_c;
    prob.oh_n = oh;
    prob.ow_n = ow;
    prob.box_w = plan.box_w;
    prob.box_h = plan.box_h;
    prob.box_n = plan.box_n;
    prob.tiles_w = (ow + plan.box_w - 1) / plan.box_w;
    prob.tiles_h = (oh + plan.box_h - 1) / plan.box_h;
    prob.c_blocks = cp / UMMA_BK;
    prob.k_w = s.k_w;
    prob.p_h = s.p_h;
    prob.p_w = s.p_w;
    prob.s_h = s.s_h;
    prob.s_w = s.s_w;
    prob.total_kb = taps * prob.c_blocks;
    prob.batch = s.batch;
    prob.out_plane = extras ? extras->out_plane : static_cast<long long>(oh) * ow;
    prob.out_off = extras ? extras->out_off : 0;
    prob.out_row = extras ? extras->out_row : ow;
    prob.out_col = extras ? extras->out_col : 1;
    prob.contig = (plan.box_w == ow && !MULTI_IMAGE && !(extras && extras->scattered)) ? 1 : 0;
    prob.vec_ok = (prob.contig && ((plan.box_h * ow) % 4 == 0) && ((oh * ow) % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(out) & 15u) == 0)) ? 1 : 0;
    // Bulk stores: contiguous tiles, plane rows of 16-byte multiples, chunk starts on 16-byte
    // boundaries (oh0 * OW is a multiple of box_h * OW), whole 32-row blocks of output channels.
    const bool bulk_store = prob.vec_ok && s.out_c % 32 == 0;
    if (bulk_store) {
        const uint64_t dims[2] = {uint64_t(oh) * ow, uint64_t(s.batch) * s.out_c};
        const uint64_t strides[1] = {uint64_t(oh) * ow * 4};
        const uint32_t box[2] = {32, 32};
        encode_tensor_map(&prob.map_out, out, 2, dims, strides, box, TmaSwizzle::B128);
    } else {
        prob.map_out = prob.map_w;
    }

    const int umma_n = plan.box_w * plan.box_h * plan.box_n;
    const int pixel_tiles = MULTI_IMAGE ? (s.batch + plan.box_n - 1) / plan.box_n
                                        : s.batch * prob.tiles_h * prob.tiles_w;
    UmmaSchedule sched = whole_tile_schedule(
        (s.out_c + UMMA_BM * CTAS - 1) / (UMMA_BM * CTAS), pixel_tiles,
        taps * prob.c_blocks, umma_n, (Cfg::A_BYTES + uint32_t(umma_n / CTAS) * UMMA_BK * 4) * CTAS * KATOMS,
        Cfg::STAGES, dev.status_word);
    // Consecutive tiles walk the output-channel tiles of one pixel block, so
    // concurrent CTAs read the same input pixels from L2.
    sched.raster_group = sched.tiles_m;
    // Tiles of several whole planes: compacted blocks of 32 channels x one plane, when a block fits
    // a warp's staging area, planes are dense and 16-byte aligned as blocks, and the plane size is
    // odd (rows of the block then fall on different shared-memory banks).
    const int plane = oh * ow, per_plane = plan.box_w * plan.box_h;
    const bool dense_planes = prob.out_plane == plane && prob.out_off == 0 && prob.out_row == ow && prob.out_col == 1;
    bool plane_store = MULTI_IMAGE && dense_planes && s.out_c % 32 == 0 && plane % 2 == 1 && plane <= 64 &&
                       per_plane % 32 == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    uint32_t staging_bytes = (bulk_store || plane_store) ? UMMA_STORE_STAGING_BYTES : 0u;
    const long long num_tiles = static_cast<long long>(sched.tiles_m) * sched.tiles_n;
    CB200_REQUIRE(num_tiles < (1LL << 30), "conv2d: too many tiles");
    // Split-K inside a cluster (one tile per cluster): see the GEMM launcher for the layout.
    int ksplit = Prob::kClusterSplit ? plan.ksplit : 1;
    // (A group's slice of the columns must hold whole planes for the compacted stores; the split
    // matters more, so they give way.)
    while (ksplit > 1 && !cluster_split_fits(umma_n, CTAS, ksplit, sched.k_blocks, KATOMS)) ksplit /= 2;
    if (plane_store && ksplit > 1 && (umma_n / ksplit) % per_plane != 0) plane_store = false;
    if (ksplit > 1 || !(bulk_store || plane_store)) staging_bytes = 0;       // split tiles stage in the idle ring
    sched.plane_store = plane_store ? 1 : 0;
    uint32_t exchange_bytes = 0;
    if (ksplit > 1) {
        int per = (sched.k_blocks + ksplit - 1) / ksplit;
        per = (per + KATOMS - 1) / KATOMS * KATOMS;
        sched.cluster_split = ksplit;
        sched.kb_per_split = per;
        exchange_bytes = uint32_t(ksplit - 1) * UMMA_BM * uint32_t(umma_n / ksplit) * 4u;
    }
    sched.exchange_bytes = exchange_bytes;
    const int fit_stages = int((Cfg::SMEM_BUDGET - staging_bytes - exchange_bytes) / Cfg::STAGE_BYTES);
    if (sched.stages > fit_stages) sched.stages = fit_stages;
    sched.tma_store = bulk_store ? 1 : 0;
    sched.ring_staging = (bulk_store && uint32_t(sched.stages) * Cfg::STAGE_BYTES >= 131072u) ? 1 : 0;
    const uint32_t smem_bytes = uint32_t(sched.stages) * Cfg::STAGE_BYTES + exchange_bytes + staging_bytes + 1024;

    long long groups = dev.num_sms / CTAS;
    if (groups < 1) groups = 1;
    if (groups > num_tiles) groups = num_tiles;
    if (ksplit > 1) groups = num_tiles;          // clusters: one per tile

    CB200_TRACE("conv2d implicit GEMM tcgen05: N=%d C=%d %dx%d -> OC=%d %dx%d, %dx%d stride %dx%d pad %dx%d; pixel box "
                "%d x %d x %d images = %d columns, ctas/mma=%d katoms=%d stages=%d clusters=%lld, K blocks=%d, "
                "cluster_split=%d, store=%s",
                s.batch, s.in_c, s.in_h, s.in_w, s.out_c, oh, ow, s.k_h, s.k_w, s.s_h, s.s_w, s.p_h, s.p_w, plan.box_w,
                plan.box_h, plan.box_n, umma_n, CTAS, KATOMS, sched.stages, groups, sched.k_blocks, ksplit,
                bulk_store ? "bulk-tensor" : plane_store ? "bulk planes" : "registers");
    auto kernel = umma_tf32_kernel<CTAS, 256, false, KATOMS, Prob>;
    UmmaEpilogueArgs epi{bias, 1, act};
    launch_umma(kernel, prob, sched, epi, groups, CTAS * ksplit, smem_bytes, Cfg::SMEM_MAX, stream);
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

}  // namespace

namespace {
// One launch: the input re-layout and, in an extra z slice of blocks, the filter packing.
void prepare_operands(const float* input, float* xt, int batch, int c, int hw, int cx, const FilterPack* filters,
                      cudaStream_t stream, const PixelScatter* scatter = nullptr) {
    // Filter packing takes as many extra z slices as give it about one block per 2048 elements
    // (small feature maps have few blocks per slice, and their filters are the large ones).
    int filter_slices = 0;
    if (filters) {
        const long long elems = static_cast<long long>(filters->oc_n) * filters->k_h *
                                (filters->row_cx > 0 ? UMMA_BK : filters->k_w * filters->cp);
        const long long per_slice = static_cast<long long>((hw + 63) / 64) * ((cx + 31) / 32);
        long long want = (elems + 2047) / 2048;
        if (want > 148 * 8) want = 148 * 8;
        filter_slices = static_cast<int>((want + per_slice - 1) / per_slice);
        if (filter_slices < 1) filter_slices = 1;
        if (filter_slices > 1024) filter_slices = 1024;
    }
    dim3 grid((hw + 63) / 64, (cx + 31) / 32, batch + filter_slices);
    CB200_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "conv2d: too many channels or images");
    const bool vec = (hw % 4 == 0) && ((reinterpret_cast<uintptr_t>(input) & 15u) == 0);
    const FilterPack f = filters ? *filters : FilterPack{};
    const int with = filters ? 1 : 0;
    if (vec && cx == 4) {
        // (The filter slices were sized for 64-pixel blocks; these blocks cover 1024 pixels, so
        // there are fewer per slice: the grid-stride loop of the packing absorbs it.)
        dim3 grid4((hw / 4 + 255) / 256, 1, batch + filter_slices);
        if (scatter) nchw_to_nhwc4_kernel<true><<<grid4, 256, 0, stream>>>(input, xt, c, hw, batch, f, with, *scatter);
        else nchw_to_nhwc4_kernel<false><<<grid4, 256, 0, stream>>>(input, xt, c, hw, batch, f, with, PixelScatter{});
        CB200_CHECK_LAUNCH();
        return;
    }
    if (scatter) {
        if (vec) nchw_to_nhwc_kernel<true, true><<<grid, 256, 0, stream>>>(input, xt, c, hw, cx, batch, f, with, *scatter);
        else nchw_to_nhwc_kernel<false, true><<<grid, 256, 0, stream>>>(input, xt, c, hw, cx, batch, f, with, *scatter);
    } else if (vec) nchw_to_nhwc_kernel<true><<<grid, 256, 0, stream>>>(input, xt, c, hw, cx, batch, f, with);
    else nchw_to_nhwc_kernel<false><<<grid, 256, 0, stream>>>(input, xt, c, hw, cx, batch, f, with);
    CB200_CHECK_LAUNCH();
}
}  // namespace

void nchw_to_nhwc(const float* input, float* xt, int batch, int c, int hw, int cx, cudaStream_t stream) {
    prepare_operands(input, xt, batch, c, hw, cx, nullptr, stream);
}

void nchw_to_nhwc_padded(const float* input, float* xt, int batch, int c, int h, int w, int cx, int pad_w,
                         cudaStream_t stream) {
    const int wp_pixels = w + 2 * pad_w;
    CB200_CUDA(cudaMemsetAsync(xt, 0, static_cast<size_t>(batch) * h * wp_pixels * cx * sizeof(float), stream));
    const PixelScatter scatter{w, wp_pixels, h * wp_pixels, 1, 1, pad_w};
    prepare_operands(input, xt, batch, c, h * w, cx, nullptr, stream, &scatter);
}

bool conv2d_igemm_supported(const ConvShape& s) {
    if (device_info().cc_major != 10) return false;
    if (s.s_h < 1 || s.s_w < 1 || s.s_h > 8 || s.s_w > 8) return false;     // TMA element strides go up to 8
    if (s.p_h >= s.k_h || s.p_w >= s.k_w) return false;     // keeps every box start within TMA's signed range
    const int oh = s.out_h(), ow = s.out_w();
    if (oh < 1 || ow < 1) return false;
    // Worth a 128-row tensor-core tile only with enough channels and pixels.
    // Few input channels (a network's first layer) still pay off: every tap's channels are padded
    // to one 32-wide K block, which the tensor cores absorb far better than the direct kernel does
    // the gather (3 x 3 x 3 -> 64 on 224 x 224 images: 6.4 ms direct).
    // One or two channels waste too much of it (128 x 1 x 28 x 28, 5 x 5: 111 us against 74 us direct).
    // One or two channels are taken only when a filter row's taps share a K block.
    if (s.out_c < 32 || (s.in_c < 3 && !conv2d_igemm_row_packed(s))) return false;
    if (static_cast<long long>(s.batch) * oh * ow < 64) return false;
    return true;
}

// Few input channels: a filter row's KW taps of cx channels fit one 32-wide K block, so the
// reduction takes KH blocks instead of KH * KW (a 7 x 7 filter over 3 channels: 7 blocks of which
// 21 / 32 are real, against 49 blocks of which 3 / 32 are).
bool conv2d_igemm_row_packed(const ConvShape& s) {
    return s.k_w > 1 && round_up(s.in_c, 4) * s.k_w <= UMMA_BK;
}

size_t conv2d_igemm_scratch_bytes(const ConvShape& s, size_t* nhwc_bytes, size_t* filter_bytes) {
    const int cx = round_up(s.in_c, 4);
    const int cp = round_up(s.in_c, UMMA_BK);
    // The larger of the two layouts (a call with flipped filters never packs rows).
    const size_t a = static_cast<size_t>(s.batch) * s.in_h * (s.in_w + 2 * s.p_w) * cx * sizeof(float);
    const size_t b = static_cast<size_t>(s.out_c) * s.k_h * s.k_w * cp * sizeof(float);
    // Both regions start on 1 KiB boundaries.
    const size_t a_pad = (a + 1023) / 1024 * 1024;
    const size_t b_pad = (b + 1023) / 1024 * 1024;
    if (nhwc_bytes) *nhwc_bytes = a_pad;
    if (filter_bytes) *filter_bytes = b_pad;
    return a_pad + b_pad;
}

namespace {
// CUDEEP_B200_CONV_ROWS=0 keeps 3 x 3 layers on the tap-per-K-block form (read once).
bool rows_form_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("CUDEEP_B200_CONV_ROWS");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

// Picks the pixel box (one image's rows, or several whole images for small maps) and the CTA
// grouping, and launches the matching kernel instantiation.
void plan_and_launch(const float* xt, const float* wp, const float* bias, float* output, const ConvShape& s,
                     int cx, int cp, int act, int force_ctas, bool row_packed, cudaStream_t stream,
                     const ConvExtras* extras) {
    const int oh = s.out_h(), ow = s.out_w();
    int ctas = force_ctas;
    if (ctas == 0) ctas = (s.out_c > UMMA_BM) ? 2 : 1;
    if (!row_packed && rows_form_enabled() && small_map_form_applies(s, ctas, output, extras == nullptr)) {
        launch_conv_small_maps(xt, wp, bias, output, s, cx, cp, act, stream);
        return;
    }
    if (!row_packed && rows_form_enabled()) {
        const RowPlan rows = plan_rows(s, ctas, output, extras == nullptr);
        if (rows.rows_per_half > 0) {
            if (ctas == 2) launch_conv_rows<2>(xt, wp, bias, output, s, cx, cp, rows, act, stream);
            else launch_conv_rows<1>(xt, wp, bias, output, s, cx, cp, rows, act, stream);
            return;
        }
    }
    TilePlan plan = plan_tile(oh, ow, ctas, s.s_h, s.s_w);
    if (plan.box_w == 0 && ctas == 2) {
        ctas = 1;
        plan = plan_tile(oh, ow, 1, s.s_h, s.s_w);
    }
    CB200_REQUIRE(plan.box_w > 0, "conv2d: no tile shape fits this output size");
    // A CTA pair stages at most 32 KB per K block, so two blocks share a pipeline
    // stage and the barrier handshake is paid half as often.
    if (!row_packed)
        plan = plan_multi_image_tile(oh, ow, s.batch, ctas, s.s_h, s.s_w, (s.out_c + UMMA_BM * ctas - 1) / (UMMA_BM * ctas),
                                     device_info().num_sms, s.k_h * s.k_w * (cp / UMMA_BK), plan);
    CB200_REQUIRE(plan.box_w > 0, "conv2d: no tile shape fits this output size");
    if (row_packed) {
        if (ctas == 2) launch_conv<2, 2, true, false>(xt, wp, bias, output, s, cx, cp, plan, act, stream, extras);
        else launch_conv<1, 1, true, false>(xt, wp, bias, output, s, cx, cp, plan, act, stream, extras);
    } else if (plan.box_n > 1) {
        if (ctas == 2) launch_conv<2, 2, false, true>(xt, wp, bias, output, s, cx, cp, plan, act, stream, extras);
        else launch_conv<1, 1, false, true>(xt, wp, bias, output, s, cx, cp, plan, act, stream, extras);
    } else {
        if (ctas == 2) launch_conv<2, 2, false, false>(xt, wp, bias, output, s, cx, cp, plan, act, stream, extras);
        else launch_conv<1, 1, false, false>(xt, wp, bias, output, s, cx, cp, plan, act, stream, extras);
    }
}
}  // namespace

bool conv2d_igemm_takes_nhwc_input(const float* input, const ConvShape& s) {
    // The kernel's own input layout is NHWC with the channel count a multiple of 4 and 16-byte
    // aligned pixels; the row-packed form (a first layer's few channels) re-lays its input with
    // padding columns and has no use for it.
    return conv2d_igemm_supported(s) && s.in_c % 4 == 0 && (reinterpret_cast<uintptr_t>(input) & 15u) == 0 &&
           !conv2d_igemm_row_packed(s);
}

void conv2d_igemm_with_scratch(const float* input, const float* weight, const float* bias,
                               float* output, const ConvShape& s, int act, void* scratch,
                               int force_ctas, cudaStream_t stream, bool flipped_filters,
                               const InputDilation* dilation, bool input_is_nhwc) {
    check_conv_shape(s);
    CB200_REQUIRE(conv2d_igemm_supported(s), "conv2d: shape not supported by the tensor-core path");
    CB200_REQUIRE(scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0,
                  "conv2d: scratch must be 256-byte aligned");
    const int cx = round_up(s.in_c, 4);
    const int cp = round_up(s.in_c, UMMA_BK);
    const int hw = s.in_h * s.in_w;
    const int taps = s.k_h * s.k_w;
    size_t nhwc_bytes = 0;
    conv2d_igemm_scratch_bytes(s, &nhwc_bytes, nullptr);
    float* xt = static_cast<float*>(scratch);
    // With a channels-last input there is no copy of it: the scratch holds the packed filters only.
    float* wp = reinterpret_cast<float*>(static_cast<char*>(scratch) + (input_is_nhwc ? 0 : nhwc_bytes));

    const bool row_packed = !flipped_filters && dilation == nullptr && conv2d_igemm_row_packed(s);
    if (input_is_nhwc) {
        CB200_REQUIRE(!flipped_filters && dilation == nullptr && conv2d_igemm_takes_nhwc_input(input, s),
                      "conv2d: an NHWC input needs C % 4 == 0, a 16-byte aligned pointer and a shape on the "
                      "tensor-core path");
        xt = const_cast<float*>(input);        // read in place: no re-layout pass, no copy
    }
    const FilterPack filters{weight, wp, s.out_c, s.in_c, s.k_h, s.k_w, cp, flipped_filters ? 1 : 0,
                             row_packed ? cx : 0};
    if (input_is_nhwc) {
        prepare_operands(nullptr, nullptr, /*batch=*/0, s.in_c, hw, cx, &filters, stream);      // filters only
    } else if (row_packed) {
        // The copy gets pad_w zero pixels on either side of every row, so that each output
        // column's window of KW pixels is contiguous in it.
        const int wp_pixels = s.in_w + 2 * s.p_w;
        CB200_CUDA(cudaMemsetAsync(xt, 0, static_cast<size_t>(s.batch) * s.in_h * wp_pixels * cx * sizeof(float),
                                   stream));
        const PixelScatter scatter{s.in_w, wp_pixels, s.in_h * wp_pixels, 1, 1, s.p_w};
        prepare_operands(input, xt, s.batch, s.in_c, hw, cx, &filters, stream, &scatter);
    } else if (dilation) {
        const InputDilation& d = *dilation;
        CB200_REQUIRE(d.d_h >= 1 && d.d_w >= 1 && d.src_h >= 1 && d.src_w >= 1 &&
                          (d.src_h - 1) * d.d_h < s.in_h && (d.src_w - 1) * d.d_w < s.in_w,
                      "conv2d: the dilated input does not fit the plane");
        CB200_CUDA(cudaMemsetAsync(xt, 0, static_cast<size_t>(s.batch) * hw * cx * sizeof(float), stream));
        const PixelScatter scatter{d.src_w, s.in_w, hw, d.d_h, d.d_w, 0};
        prepare_operands(input, xt, s.batch, s.in_c, d.src_h * d.src_w, cx, &filters, stream, &scatter);
    } else {
        prepare_operands(input, xt, s.batch, s.in_c, hw, cx, &filters, stream);
    }

    plan_and_launch(xt, wp, bias, output, s, cx, cp, act, force_ctas, row_packed, stream, nullptr);
}

void conv2d_igemm(const float* input, const float* weight, const float* bias, float* output,
                  const ConvShape& s, int act, cudaStream_t stream, bool flipped_filters,
                  const InputDilation* dilation, bool input_is_nhwc) {
    size_t filter_bytes = 0;
    size_t bytes = conv2d_igemm_scratch_bytes(s, nullptr, &filter_bytes);
    if (input_is_nhwc) bytes = filter_bytes;
    // Stream-ordered scratch, as the reference does for its temporaries
    // (conv_kernel.cu:282,314,748-754): safe when calls on several streams overlap.
    void* scratch = scratch_alloc(bytes, stream);
    try {
        conv2d_igemm_with_scratch(input, weight, bias, output, s, act, scratch, 0, stream, flipped_filters,
                                  dilation, input_is_nhwc);
    } catch (...) {
        scratch_free(scratch, stream);
        throw;
    }
    scratch_free(scratch, stream);
}

// ------------------------------------------------------------------ grad_input of a strided layer
//
// dx[n,c,ih,iw] = sum over (oc, kh, kw) with (ih + p - kh) divisible by s of
//                 dy[n,oc,(ih + p - kh) / s, ...] * w[oc,c,kh,kw].
// Input pixels fall into s_h * s_w classes by ((ih + p_h) mod s_h, (iw + p_w) mod s_w).  Class (a, b)
// is reached only by the taps kh = a + s_h * j, kw = b + s_w * l, and with ih = s_h * u + a - p_h its
// values are  sum_{oc,j,l} dy[n,oc,u - j,v - l] * w[oc,c,a + s_h*j,b + s_w*l]:  a stride-1
// convolution of dy itself with the reversed sub-filter.  All classes together are ONE stride-1
// convolution of dy with ceil(KH / s_h) x ceil(KW / s_w) taps and s_h * s_w * C output channels (a
// class's missing taps are zero filters), followed by a pass that weaves the classes' planes into dx -
// the sub-pixel form of a transposed convolution.  No zeros are inserted into dy, so the tensor cores
// do ceil(KH/s_h)*ceil(KW/s_w)*s_h*s_w / (KH*KW) of the useful work (16/9 for 3 x 3 stride 2) instead
// of s_h*s_w times it, and the class axis fills the 128 accumulator rows that C alone may not.
namespace {
// One axis of the plan.  Class a's pixels are ih = s*u + a - p for u in [lo[a], hi[a]]; its plane row
// u' = u - lo[a] is  sum_j dy[u' + lo[a] - j] * w[a + s*j]  over its taps j in [0, taps[a]).  With
// j'' = j - lo[a] every class reads dy[u' - j''] for j'' in [j_min, j_max]: one stride-1 correlation
// with j_max - j_min + 1 taps and padding j_max, whose tap t is j'' = j_max - t.
struct AxisPlan {
    int lo[8];
    int taps;      // of the combined filter
    int pad;       // = j_max
    int extent;    // plane rows (columns): the largest class's
    bool ok;
};

int ceil_div_int(int a, int b) { return (a + b - 1) / b; }

AxisPlan plan_axis(int extent, int k, int s, int p) {
    AxisPlan ax{};
    int j_min = 0, j_max = -(1 << 30);
    ax.extent = 0;
    ax.ok = false;
    for (int a = 0; a < s; ++a) {
        ax.lo[a] = p > a ? ceil_div_int(p - a, s) : 0;
        const int hi = (extent - 1 + p - a) >= 0 ? (extent - 1 + p - a) / s : -1;
        const int class_taps = a < k ? ceil_div_int(k - a, s) : 0;
        if (hi < ax.lo[a]) {            // no pixel of this class exists
            ax.lo[a] = 0;
            continue;
        }
        if (hi - ax.lo[a] + 1 > ax.extent) ax.extent = hi - ax.lo[a] + 1;
        if (class_taps == 0) continue;  // its pixels get no gradient: all of its taps pack as zero
        if (-ax.lo[a] < j_min) j_min = -ax.lo[a];
        if (class_taps - 1 - ax.lo[a] > j_max) j_max = class_taps - 1 - ax.lo[a];
        ax.ok = true;
    }
    if (!ax.ok) return ax;
    if (j_max < 0) j_max = 0;
    ax.taps = j_max - j_min + 1;
    ax.pad = j_max;
    return ax;
}

struct ParityPlan {
    AxisPlan h, w;
    int cols_padded;       // plane pitch: columns rounded up to 4 so that rows stay 16-byte multiples
    ConvShape sub;         // the stride-1 convolution over dy
};

ParityPlan make_parity_plan(const ConvShape& s) {
    ParityPlan p{};
    p.h = plan_axis(s.in_h, s.k_h, s.s_h, s.p_h);
    p.w = plan_axis(s.in_w, s.k_w, s.s_w, s.p_w);
    if (!p.h.ok || !p.w.ok) return p;
    p.cols_padded = (p.w.extent + 3) / 4 * 4;
    // The input extent is chosen so that the stride-1 output size is exactly rows x padded columns;
    // the tensor map keeps dy's true extent, so whatever lies outside it reads as zero.
    p.sub = ConvShape{s.batch, s.out_c, s.in_c * s.s_h * s.s_w, p.h.extent + p.h.taps - 1 - 2 * p.h.pad,
                      p.cols_padded + p.w.taps - 1 - 2 * p.w.pad, p.h.taps, p.w.taps, 1, 1, p.h.pad, p.w.pad};
    return p;
}

size_t round_1k(size_t v) { return (v + 1023) / 1024 * 1024; }

// grad_input[n][c][ih][iw] = planes[n][(a * s_w + b) * C + c][u - lo_h[a]][v - lo_w[b]] with (a, u) from
// ih + p_h and (b, v) from iw + p_w.  One thread writes four consecutive pixels of a row (one 128-bit
// store when rows are 16-byte multiples).
struct WeaveArgs {
    int c, h, w, s_h, s_w, p_h, p_w, rows, pitch;
    PackedInts8 lo_h, lo_w;
};

// SH, SW: the strides as compile-time constants (0: read them from the arguments), so that the
// divisions by them are shifts or multiplications.  blockIdx.y is the (image, channel) plane.
// PER: output pixels per thread (4, or 8 for rows that are multiples of 8: twice the loads in flight).
template <bool VEC, int SH, int SW, int PER = 4>
__global__ void __launch_bounds__(256)
weave_parity_classes_kernel(const float* __restrict__ planes, float* __restrict__ dx, WeaveArgs t) {
    const int s_h = SH > 0 ? SH : t.s_h, s_w = SW > 0 ? SW : t.s_w;
    const int groups = (t.w + PER - 1) / PER;
    const int work = t.h * groups;
    const long long plane_px = static_cast<long long>(t.rows) * t.pitch;
    const int n = blockIdx.y / t.c, c = blockIdx.y - n * t.c;
    // planes of this image: [class][channel]; class stride is C planes
    const float* src0 = planes + (static_cast<long long>(n) * s_h * s_w * t.c + c) * plane_px;
    const long long class_stride = static_cast<long long>(t.c) * plane_px;
    float* dst0 = dx + static_cast<long long>(blockIdx.y) * t.h * t.w;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < work; idx += gridDim.x * blockDim.x) {
        const int ih = idx / groups, g = idx - ih * groups;
        const int a = (ih + t.p_h) % s_h;
        const int u = (ih + t.p_h) / s_h - t.lo_h[a];
        const float* row = src0 + static_cast<long long>(a) * s_w * class_stride + static_cast<long long>(u) * t.pitch;
        float v[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int iw = g * PER + j;
            const int b = (iw + t.p_w) % s_w;
            const int q = (iw + t.p_w) / s_w - t.lo_w[b];
            v[j] = iw < t.w ? __ldg(row + b * class_stride + q) : 0.0f;
        }
        float* dst = dst0 + static_cast<long long>(ih) * t.w + g * PER;
        if (VEC) {
#pragma unroll
            for (int j = 0; j < PER; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < PER; ++j)
                if (g * PER + j < t.w) dst[j] = v[j];
        }
    }
}

template <bool VEC>
void launch_weave(const float* planes, float* dx, const WeaveArgs& t, long long n_planes, cudaStream_t stream) {
    const bool eight = VEC && t.w % 8 == 0 && t.s_h == 2 && t.s_w == 2;
    const int work = t.h * ((t.w + (eight ? 7 : 3)) / (eight ? 8 : 4));
    int bx = (work + 255) / 256;
    if (bx > 64) bx = 64;
    // gridDim.y is limited to 65535: whole images per launch (blockIdx.y = image * C + channel).
    CB200_REQUIRE(t.c <= 65535, "conv2d grad_input: too many channels");
    const long long chunk = static_cast<long long>(65535 / t.c) * t.c;
    for (long long first = 0; first < n_planes; first += chunk) {
        const long long count = n_planes - first < chunk ? n_planes - first : chunk;
        const dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(count));
        const WeaveArgs& args = t;
        const float* src = planes + (first / t.c) * t.s_h * t.s_w * t.c * static_cast<long long>(t.rows) * t.pitch;
        float* dst = dx + first * static_cast<long long>(t.h) * t.w;
        if (eight) weave_parity_classes_kernel<VEC, 2, 2, 8><<<grid, 256, 0, stream>>>(src, dst, args);
        else if (t.s_h == 2 && t.s_w == 2) weave_parity_classes_kernel<VEC, 2, 2><<<grid, 256, 0, stream>>>(src, dst, args);
        else if (t.s_h == 3 && t.s_w == 3) weave_parity_classes_kernel<VEC, 3, 3><<<grid, 256, 0, stream>>>(src, dst, args);
        else if (t.s_h == 4 && t.s_w == 4) weave_parity_classes_kernel<VEC, 4, 4><<<grid, 256, 0, stream>>>(src, dst, args);
        else weave_parity_classes_kernel<VEC, 0, 0><<<grid, 256, 0, stream>>>(src, dst, args);
        CB200_CHECK_LAUNCH();
    }
}
}  // namespace

bool conv2d_grad_input_by_parity_supported(const ConvShape& s) {
    if (device_info().cc_major != 10) return false;
    if (s.s_h < 1 || s.s_w < 1 || (s.s_h == 1 && s.s_w == 1) || s.s_h > 8 || s.s_w > 8) return false;
    if (s.p_h > s.k_h - 1 || s.p_w > s.k_w - 1) return false;
    if (s.out_c < 32) return false;                  // dy's channels are the reduction
    const ParityPlan p = make_parity_plan(s);
    if (!p.h.ok || !p.w.ok || p.h.extent < 1 || p.w.extent < 1 || p.sub.in_h < 1 || p.sub.in_w < 1) return false;
    if (static_cast<long long>(p.sub.out_c) > 65535) return false;
    return conv2d_igemm_supported(p.sub) && !conv2d_igemm_row_packed(p.sub);
}

void conv2d_grad_input_by_parity(const float* grad_output, const float* weight, float* grad_input,
                                 const ConvShape& s, cudaStream_t stream) {
    CB200_REQUIRE(conv2d_grad_input_by_parity_supported(s), "conv2d grad_input: shape not supported by the parity form");
    const ParityPlan p = make_parity_plan(s);
    const int oh = s.out_h(), ow = s.out_w();
    const int cx = round_up(s.out_c, 4);             // channels of the NHWC copy of dy
    const int cp = round_up(s.out_c, UMMA_BK);
    const int taps = p.h.taps * p.w.taps;
    // Scratch: [NHWC copy of grad_output][packed filters of all classes][the classes' dense planes].
    // (Storing every stride-th pixel straight from the epilogue instead of weaving dense planes was
    // measured at 201 us against 158 us for the dilated form on a 64 x 64 x 56 x 56 <- 128, 3 x 3
    // stride 2 layer: a 4-byte write per 32-byte sector.)
    const size_t nhwc_bytes = round_1k(static_cast<size_t>(s.batch) * oh * ow * cx * sizeof(float));
    const size_t filter_bytes = round_1k(static_cast<size_t>(p.sub.out_c) * taps * cp * sizeof(float));
    const size_t plane_bytes =
        round_1k(static_cast<size_t>(s.batch) * p.sub.out_c * p.h.extent * p.cols_padded * sizeof(float));
    char* scratch = static_cast<char*>(scratch_alloc(nhwc_bytes + filter_bytes + plane_bytes, stream));
    try {
        float* xt = reinterpret_cast<float*>(scratch);
        float* wp = reinterpret_cast<float*>(scratch + nhwc_bytes);
        float* planes = reinterpret_cast<float*>(scratch + nhwc_bytes + filter_bytes);
        FilterPack filters{weight, wp, p.sub.out_c, s.out_c, p.h.taps, p.w.taps, cp, 1, 0};
        filters.sub_sh = s.s_h;
        filters.sub_sw = s.s_w;
        filters.fwd_c = s.in_c;
        filters.full_kh = s.k_h;
        filters.full_kw = s.k_w;
        filters.pad_h = p.h.pad;
        filters.pad_w = p.w.pad;
        WeaveArgs args{s.in_c, s.in_h, s.in_w, s.s_h, s.s_w, s.p_h, s.p_w, p.h.extent, p.cols_padded, {}, {}};
        for (int a = 0; a < 8; ++a) {
            filters.lo_h.set(a, a < s.s_h ? p.h.lo[a] : 0);
            filters.lo_w.set(a, a < s.s_w ? p.w.lo[a] : 0);
            args.lo_h = filters.lo_h;
            args.lo_w = filters.lo_w;
        }
        prepare_operands(grad_output, xt, s.batch, s.out_c, oh * ow, cx, &filters, stream);
        ConvExtras extras;
        extras.map_h = oh;
        extras.map_w = ow;
        extras.out_plane = static_cast<long long>(p.h.extent) * p.cols_padded;
        extras.out_off = 0;
        extras.out_row = p.cols_padded;
        extras.out_col = 1;
        extras.scattered = false;
        CB200_TRACE("conv2d grad_input by parity classes: stride %dx%d, %d classes x %d channels, %dx%d taps each, "
                    "planes of %d x %d", s.s_h, s.s_w, s.s_h * s.s_w, s.in_c, p.h.taps, p.w.taps, p.h.extent, p.cols_padded);
        plan_and_launch(xt, wp, nullptr, planes, p.sub, cx, cp, EPI_NONE, 0, false, stream, &extras);
        const bool vec = s.in_w % 4 == 0 && (reinterpret_cast<uintptr_t>(grad_input) & 15u) == 0;
        const long long n_planes = static_cast<long long>(s.batch) * s.in_c;
        if (vec) launch_weave<true>(planes, grad_input, args, n_planes, stream);
        else launch_weave<false>(planes, grad_input, args, n_planes, stream);
    } catch (...) {
        scratch_free(scratch, stream);
        throw;
    }
    scratch_free(scratch, stream);
}

}  // namespace cudeep_b200
