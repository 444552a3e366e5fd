// Activation-side kernels: sign packing with the fused mean-|x| map, and the K box filter.
//
// All three are bound by HBM bandwidth: the fp32 source (4 B per element) is read exactly once
// and 1/32 (bits) or 1/4 (int8) of that is written. One thread owns one pixel and walks its
// channels in ascending order, so the mean-|x| sum is accumulated in the very order upstream
// uses (src/bcast_calculate_k.cpp:55-65) and rounds identically; with an NCHW source the 32
// lanes of a warp read 32 neighbouring pixels of one channel plane, a full 128-byte line.
#include "kernels.cuh"

#include <atomic>

namespace xb200 {

namespace {
// Source floats are read exactly once: keep them out of the L1 so that the loads in flight are
// not limited by its size (conv4 step 61.0 -> 57.0 us together with the carve-out below).
__device__ __forceinline__ float ld_stream(const float *p) {
    float v;
    asm("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}


enum OutKind { kBitsDense = 0, kBytesFramed = 2 };

struct BinArgs {
    const float *src;
    void *out;
    float *a;
    long n_px;        // mb*ih*iw
    int ic, hw, iw;   // hw = ih*iw
    long img_stride;  // elements between images in src
    long c_stride;    // elements between channels of one pixel
    long px_stride;   // elements between pixels of one image
    float inv_ic;
    int words;        // 32-bit words per packed row (icw, or icp/4 for bytes)
    int wp, hp, lead, ih;
};

__device__ __forceinline__ unsigned sign_clear(float x) { return (~__float_as_uint(x)) >> 31; }

// Row of the packed matrix that pixel (n, h, w) owns.
template <int KIND>
__device__ __forceinline__ long packed_row(const BinArgs &g, long px) {
    if (KIND == kBitsDense) return px;
    const int n = (int)(px / g.hw);
    const int r = (int)(px - (long)n * g.hw);
    const int h = r / g.iw, w = r - h * g.iw;
    return g.lead + ((long)n * g.hp + h) * g.wp + w;
}

template <int KIND, bool WITH_A, bool WITH_PACK>
__global__ void __launch_bounds__(128) binarize_kernel(const BinArgs g) {
    const long px = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (px >= g.n_px) return;
    const int n = (int)(px / g.hw);
    const int r = (int)(px - (long)n * g.hw);
    const float *p = g.src + n * g.img_stride + r * g.px_stride;
    uint32_t *row = WITH_PACK ? (uint32_t *)g.out + packed_row<KIND>(g, px) * g.words : nullptr;

    float acc = 0.f;
    const int full = g.ic & ~31;
    int c = 0;
    for (; c < full; c += 32) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = __ldg(p + (long)(c + i) * g.c_stride);
        if (WITH_A) {
#pragma unroll
            for (int i = 0; i < 32; i++) acc = __fadd_rn(acc, __fmul_rn(fabsf(v[i]), g.inv_ic));
        }
        if (WITH_PACK) {
            if (KIND == kBytesFramed) {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint32_t w = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        w |= (sign_clear(v[4 * j + i]) ? 0x01u : 0xFFu) << (8 * i);
                    row[c / 4 + j] = w;
                }
            } else {
                uint32_t w = 0;
#pragma unroll
                for (int i = 0; i < 32; i++) w = (w << 1) | sign_clear(v[i]);
                row[c / 32] = w;
            }
        }
    }
    if (c < g.ic) {  // channel tail: absent channels pack as zero
        uint32_t wbits = 0;
        uint32_t wbytes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int i = 0; i < 32; i++) {
            unsigned bit = 0;
            if (c + i < g.ic) {
                const float x = __ldg(p + (long)(c + i) * g.c_stride);
                if (WITH_A) acc = __fadd_rn(acc, __fmul_rn(fabsf(x), g.inv_ic));
                bit = sign_clear(x);
                wbytes[i / 4] |= (bit ? 0x01u : 0xFFu) << (8 * (i % 4));
            }
            wbits = (wbits << 1) | bit;
        }
        if (WITH_PACK) {
            if (KIND == kBytesFramed) {
#pragma unroll
                for (int j = 0; j < 8; j++) row[c / 4 + j] = wbytes[j];
            } else {
                row[c / 32] = wbits;
            }
        }
        c += 32;
    }
    if (WITH_PACK && KIND == kBytesFramed) {
        // chunk padding beyond the last 32-channel group stays zero
        for (int j = c / 4; j < g.words; j++) row[j] = 0u;
    }
    if (WITH_A) g.a[px] = acc;
}

// ---- NCHW source, +-1 bytes on the frame: the layout the tensor-core convolution reads -------
//
// A block of four warps owns 32 neighbouring pixels and walks the channels in chunks of 128.
// All warps load (lane = pixel, warp w the w-th quarter of the chunk's channels, so a load
// instruction reads one 128-byte line of a channel plane; 32 independent loads per thread, issued
// one chunk ahead so that they are in flight while the previous chunk is consumed). |x|/IC goes to a float tile and the sign byte to a byte
// tile in shared memory. Warp 0 then adds the float tile up channel by channel, one lane per
// pixel, which keeps upstream's summation order, while the other warps copy the byte tile out
// as one coalesced 128-byte line per pixel. Seven blocks are resident per SM (72 registers per
// thread, and the shared-memory carve-out is sized to match).
//
// TPER = channels per warp and chunk = loads per thread and chunk: 32 (chunks of 128 channels)
// or 24 (chunks of 96), the latter for channel counts that are a multiple of 96 but not of 128
// (AlexNet conv2), where a 128-channel chunk would leave a quarter of the threads without work.
// Bytes past the last channel of a packed row are never written: they are zero from allocation.
constexpr int TPX = 32;    // pixels per block
constexpr int TWARPS = 4;

template <bool WITH_A, bool WITH_PACK, int TPER>
__global__ void __launch_bounds__(TWARPS * 32) binarize_bytes_nchw_kernel(const BinArgs g) {
    constexpr int TCC = TPER * TWARPS;  // channels per chunk
    constexpr int TLD = TCC + 4;
    __shared__ float f_s[WITH_A ? TCC * TPX : 1];
    __shared__ __align__(16) uint8_t b_s[WITH_PACK ? TPX * TLD : 4];
    __shared__ long row_s[TPX];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // The dependent grid (the convolution) may be launched once every block of this grid has
    // got this far, i.e. when none is waiting for an SM any more; its CTAs then move in as SMs
    // drain and set themselves up under this grid's tail (conv4 step 56.6 -> 55.5 us against
    // triggering at the end of the block). They wait for this grid's results themselves.
    dependency_release();
    dependency_wait();  // nothing of an earlier kernel is read or overwritten before this
    const long px = (long)blockIdx.x * TPX + lane;
    const bool live = px < g.n_px;
    const int n = live ? (int)(px / g.hw) : 0;
    const int r = live ? (int)(px - (long)n * g.hw) : 0;
    const float *p = g.src + n * g.img_stride + r;
    if (warp == 0) row_s[lane] = live ? packed_row<kBytesFramed>(g, px) : -1;

    // channel extent walked: the channels, rounded up to whole 32-bit words of the packed row
    const int c_end = WITH_PACK ? min(g.words * 4, (g.ic + 3) & ~3) : g.ic;
    float acc = 0.f;
    // Warp w owns the 32 consecutive channels [32w, 32w+32) of every chunk, so four of its sign
    // bytes make one 32-bit word of the packed row.
    const float *pw = p + (long)(TPER * warp) * g.hw;
    const int cw = TPER * warp;  // first channel of this warp inside a chunk
    float v[TPER];
    if (live && TCC <= g.ic) {
#pragma unroll
        for (int i = 0; i < TPER; i++) v[i] = ld_stream(pw + (long)i * g.hw);
    } else {
#pragma unroll
        for (int i = 0; i < TPER; i++)
            v[i] = (live && cw + i < g.ic) ? ld_stream(pw + (long)i * g.hw) : 0.f;
    }
    for (int c0 = 0; c0 < c_end; c0 += TCC) {
        const bool full = c0 + TCC <= g.ic;  // no channel tail in this chunk
        if (WITH_A) {
#pragma unroll
            for (int i = 0; i < TPER; i++)
                f_s[(cw + i) * TPX + lane] = __fmul_rn(fabsf(v[i]), g.inv_ic);
        }
        if (WITH_PACK) {
            uint32_t *brow = reinterpret_cast<uint32_t *>(b_s + lane * TLD) + cw / 4;
#pragma unroll
            for (int j = 0; j < TPER / 4; j++) {
                // sign bit set -> 0xFF (-1), clear -> 0x01 (+1): 0x01 ^ (sign * 0xFE) per byte
                const uint32_t m = (__float_as_uint(v[4 * j]) >> 31) |
                                   ((__float_as_uint(v[4 * j + 1]) >> 31) << 8) |
                                   ((__float_as_uint(v[4 * j + 2]) >> 31) << 16) |
                                   ((__float_as_uint(v[4 * j + 3]) >> 31) << 24);
                uint32_t word = 0x01010101u ^ (m * 0xFEu);
                if (!full) {  // channels past the last one are zero bytes
                    const int left = g.ic - (c0 + cw + 4 * j);
                    word = left >= 4 ? word : left <= 0 ? 0u : (word & (0xFFFFFFFFu >> (8 * (4 - left))));
                }
                brow[j] = word;
            }
        }
        __syncthreads();
        if (c0 + TCC < c_end) {  // next chunk's loads fly while this one is consumed
            const float *pn = pw + (long)(c0 + TCC) * g.hw;
            if (live && c0 + 2 * TCC <= g.ic) {
#pragma unroll
                for (int i = 0; i < TPER; i++) v[i] = ld_stream(pn + (long)i * g.hw);
            } else {
#pragma unroll
                for (int i = 0; i < TPER; i++)
                    v[i] = (live && c0 + TCC + cw + i < g.ic) ? ld_stream(pn + (long)i * g.hw) : 0.f;
            }
        }
        if (WITH_A && warp == 0) {
            const int nc = min(TCC, g.ic - c0);
            if (nc == TCC) {
#pragma unroll
                for (int j0 = 0; j0 < TCC; j0 += 16) {
                    float t[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) t[j] = f_s[(j0 + j) * TPX + lane];
#pragma unroll
                    for (int j = 0; j < 16; j++) acc = __fadd_rn(acc, t[j]);
                }
            } else {
                // channel tail: same order, groups of 16 loads in flight while they fit
                int j0 = 0;
                for (; j0 + 16 <= nc; j0 += 16) {
                    float t[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) t[j] = f_s[(j0 + j) * TPX + lane];
#pragma unroll
                    for (int j = 0; j < 16; j++) acc = __fadd_rn(acc, t[j]);
                }
                for (; j0 < nc; j0++) acc = __fadd_rn(acc, f_s[j0 * TPX + lane]);
            }
        } else if (WITH_PACK) {
            // a warp writes one pixel per pass: 32 lanes x 4 bytes, one 128-byte line
            const int first = WITH_A ? warp - 1 : warp, step = WITH_A ? TWARPS - 1 : TWARPS;
            const int nwords = (min(TCC, c_end - c0) + 3) / 4;
            constexpr int WPP = TCC / 4;   // 32-bit words per pixel and chunk
            constexpr int PPW = 32 / WPP;  // pixels a warp writes per pass
            const int half = lane / WPP, wl = lane % WPP;
            for (int pi = PPW * first + half; pi < TPX; pi += PPW * step) {
                const long row = row_s[pi];
                if (row >= 0 && wl < nwords && half < PPW)
                    ((uint32_t *)g.out)[row * g.words + c0 / 4 + wl] =
                        *reinterpret_cast<const uint32_t *>(&b_s[pi * TLD + 4 * wl]);
            }
        }
        __syncthreads();
    }
    if (WITH_A && warp == 0 && live) g.a[px] = acc;
}

struct BoxArgs {
    const float *a;
    float *k;
    long n_out;
    int ih, iw, oh, ow, kh, kw, sh, sw, ph, pw;
    float inv_khw;
};

__global__ void __launch_bounds__(256) box_filter_kernel(const BoxArgs g) {
    const long o = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= g.n_out) return;
    const int ohw = g.oh * g.ow;
    const int n = (int)(o / ohw);
    const int r = (int)(o - (long)n * ohw);
    const int oh = r / g.ow, ow = r - oh * g.ow;
    const float *img = g.a + (long)n * g.ih * g.iw;
    float acc = 0.f;
    for (int kh = 0; kh < g.kh; kh++) {
        const int ih = oh * g.sh - g.ph + kh;
        if (ih < 0 || ih >= g.ih) continue;
        for (int kw = 0; kw < g.kw; kw++) {
            const int iw = ow * g.sw - g.pw + kw;
            if (iw < 0 || iw >= g.iw) continue;
            acc = __fadd_rn(acc, __fmul_rn(__ldg(img + ih * g.iw + iw), g.inv_khw));
        }
    }
    g.k[o] = acc;
}

BinArgs bin_args(const Plan &p, const float *src, void *out, float *a) {
    BinArgs g;
    g.src = src; g.out = out; g.a = a;
    g.n_px = (long)p.mb * p.ih * p.iw;
    g.ic = p.ic; g.hw = p.ih * p.iw; g.iw = p.iw; g.ih = p.ih;
    g.img_stride = (long)p.ic * p.ih * p.iw;
    g.c_stride = p.src_nhwc ? 1 : (long)p.ih * p.iw;
    g.px_stride = p.src_nhwc ? p.ic : 1;
    g.inv_ic = p.inv_ic;
    g.words = p.family == kTcgen05 ? p.icp / 4 : p.icw;
    g.wp = p.wp; g.hp = p.hp; g.lead = p.lead;
    return g;
}

constexpr int kResidentBlocks = 7;  // tiled kernel: blocks per SM the carve-out is sized for

template <bool WITH_A, bool WITH_PACK>
cudaError_t launch_bin(const Plan &p, const BinArgs &g, cudaStream_t s) {
    const int threads = 128;
    const unsigned blocks = (unsigned)((g.n_px + threads - 1) / threads);
    if (blocks == 0) return cudaSuccess;
    if (!p.src_nhwc && (p.family == kTcgen05 || !WITH_PACK)) {
        // Shared-memory carve-out sized for kResidentBlocks blocks per SM, once per device. Left
        // to itself the driver sizes it for as many blocks as the thread count allows, which
        // leaves the L1 too small for the loads in flight; a kernel that streams with 32 loads
        // per thread outstanding does not need that many warps. Measured on conv4, minibatch 256:
        // the pass with the mean-|x| map 20.9 -> 19.1 us, and the convolution that follows starts
        // about 3 us earlier (whole step 65.5 -> 60.4 us).
        static std::atomic<bool> tuned[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (!tuned[dev & 63].exchange(true, std::memory_order_acq_rel)) {
            const int blocks = kResidentBlocks;
            cudaFuncAttributes fa;
            int smem_sm = 0;
            if (blocks > 0 &&
                cudaFuncGetAttributes(&fa, binarize_bytes_nchw_kernel<WITH_A, WITH_PACK, 32>) == cudaSuccess &&
                cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess &&
                smem_sm > 0) {
                long pct = (100L * blocks * ((long)fa.sharedSizeBytes + 1024) + smem_sm - 1) / smem_sm;
                if (pct > 100) pct = 100;
                cudaFuncSetAttribute(binarize_bytes_nchw_kernel<WITH_A, WITH_PACK, 32>,
                                     cudaFuncAttributePreferredSharedMemoryCarveout, (int)pct);
                cudaFuncSetAttribute(binarize_bytes_nchw_kernel<WITH_A, WITH_PACK, 24>,
                                     cudaFuncAttributePreferredSharedMemoryCarveout, (int)pct);
            }
            (void)cudaGetLastError();
        }
        note_launch();
        // Launched with programmatic stream serialisation like the convolution: behind one of
        // this library's kernels (which trigger early) the blocks become resident while it
        // drains and wait in dependency_wait(); behind anything else nothing changes.
        const dim3 grid((unsigned)((g.n_px + TPX - 1) / TPX)), block(TWARPS * 32);
        if (g.ic % 96 == 0 && g.ic % 128 != 0)
            return launch_overlapped(binarize_bytes_nchw_kernel<WITH_A, WITH_PACK, 24>, grid, block,
                                     0, s, 1, g);
        return launch_overlapped(binarize_bytes_nchw_kernel<WITH_A, WITH_PACK, 32>, grid, block, 0,
                                 s, 1, g);
    }
    switch (p.family) {
        case kPopc: binarize_kernel<kBitsDense, WITH_A, WITH_PACK><<<blocks, threads, 0, s>>>(g); break;
        default: binarize_kernel<kBytesFramed, WITH_A, WITH_PACK><<<blocks, threads, 0, s>>>(g); break;
    }
    note_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_binarize_data(const Plan &p, const float *src, void *bin_src, float *a,
                                 cudaStream_t s) {
    const BinArgs g = bin_args(p, src, bin_src, a);
    return a ? launch_bin<true, true>(p, g, s) : launch_bin<false, true>(p, g, s);
}

cudaError_t launch_mean_abs(const Plan &p, const float *src, float *a, cudaStream_t s) {
    const BinArgs g = bin_args(p, src, nullptr, a);
    return launch_bin<true, false>(p, g, s);
}

cudaError_t launch_box_filter(const Plan &p, const float *a, float *k, cudaStream_t s) {
    BoxArgs g;
    g.a = a; g.k = k;
    g.n_out = (long)p.mb * p.oh * p.ow;
    g.ih = p.ih; g.iw = p.iw; g.oh = p.oh; g.ow = p.ow; g.kh = p.kh; g.kw = p.kw;
    g.sh = p.sh; g.sw = p.sw; g.ph = p.ph; g.pw = p.pw;
    g.inv_khw = p.inv_khw;
    const int threads = 256;
    const unsigned blocks = (unsigned)((g.n_out + threads - 1) / threads);
    if (blocks == 0) return cudaSuccess;
    box_filter_kernel<<<blocks, threads, 0, s>>>(g);
    note_launch();
    return cudaGetLastError();
}

}  // namespace xb200
