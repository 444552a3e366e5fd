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
// one chunk ahead so that they are in flight while the previous chunk is consumed). |x|/IC goes
// to a float tile and the sign byte to a byte tile in shared memory, both pixel-major. Warp 0 then
// adds the float tile up channel by channel, one lane per pixel, which keeps upstream's summation
// order, while the other warps copy the byte tile out, 8 bytes per lane, a pixel's 128-byte line
// per half warp. Five blocks are resident per SM (nine of the 96-channel kind): the shared-memory
// carve-out is sized for that, see launch_bin().
//
// The kernel is as much bound by instruction issue as by memory (a profile of the first version
// on the 96-channel AlexNet layer: 29 instructions issued per global load, the schedulers busy
// in 69 % of the active cycles, DRAM at 31 %). Hence: the sign bytes of four floats come from
// three byte permutes and one logic operation; both tiles are written and read with 8- and
// 16-byte shared-memory accesses, their rows padded so that these stay free of bank conflicts;
// pixel coordinates are 32-bit (the host sends anything larger to the generic kernel).
//
// TPER = channels per warp and chunk = loads per thread and chunk: 32 (chunks of 128 channels)
// or 24 (chunks of 96), the latter for channel counts that are a multiple of 96 but not of 128
// (AlexNet conv2), where a 128-channel chunk would leave a quarter of the threads without work.
// Bytes past the last channel of a packed row are zero from allocation, and only zeros are
// ever written there.
constexpr int TPX = 32;    // pixels per block
constexpr int TWARPS = 4;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// The +-1 bytes of four floats, the first in the lowest byte: sign bit set -> 0xFF, clear -> 0x01.
// A selector nibble of 0xB / 0xF replicates the top bit of byte 3 of the first / second operand.
__device__ __forceinline__ uint32_t sign_bytes(float a, float b, float c, float d) {
    const uint32_t ab = prmt(__float_as_uint(a), __float_as_uint(b), 0xFBFBu);
    const uint32_t cd = prmt(__float_as_uint(c), __float_as_uint(d), 0xFBFBu);
    return (prmt(ab, cd, 0x5410u) & 0xFEFEFEFEu) ^ 0x01010101u;
}

// Element i of a column of floats whose rows are `pitch` bytes apart. The plain expression on
// 64-bit element offsets compiled to seven integer instructions per load; 32-bit byte offsets to
// about five; WIDE states the address as the one 32 x 32 + 64-bit multiply-add it is. Measured
// on the pass with the mean-|x| map: 128-channel chunks 16.7-17.0 -> 15.5 us on conv4 (whole step
// 50.6 -> 49.5 us), 21.7 -> 21.2 on the VGG layer; 96-channel chunks 9.3 -> 9.6 us on conv2, so
// that kernel keeps the plain form.
template <bool WIDE>
__device__ __forceinline__ const float *row_ptr(const float *p, unsigned i, unsigned pitch) {
    if (WIDE) {
        unsigned long long d;
        asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(d) : "r"(i), "r"(pitch), "l"(p));
        return reinterpret_cast<const float *>(d);
    }
    return reinterpret_cast<const float *>(reinterpret_cast<const char *>(p) + (size_t)(i * pitch));
}

template <bool WITH_A, bool WITH_PACK, int TPER>
__global__ void __launch_bounds__(TWARPS * 32) binarize_bytes_nchw_kernel(const BinArgs g) {
    constexpr int TCC = TPER * TWARPS;  // channels per chunk
    constexpr int FLD = TCC + 4;        // floats per pixel of the float tile
    constexpr int TLD = TCC + 8;        // bytes per pixel of the byte tile
    __shared__ __align__(16) float f_s[WITH_A ? TPX * FLD : 4];
    __shared__ __align__(16) uint8_t b_s[WITH_PACK ? TPX * TLD : 8];
    __shared__ long row_s[TPX];  // a pixel's packed row, as an offset in units of 8 bytes

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // The dependent grid (the convolution) may be launched once every block of this grid has
    // got this far, i.e. when none is waiting for an SM any more; its CTAs then move in as SMs
    // drain and set themselves up under this grid's tail (conv4 step 56.6 -> 55.5 us against
    // triggering at the end of the block). They wait for this grid's results themselves.
    dependency_release();
    dependency_wait();  // nothing of an earlier kernel is read or overwritten before this
    const unsigned px = blockIdx.x * TPX + lane;
    const bool live = px < (unsigned)g.n_px;
    const int n_live = (int)min((unsigned)TPX, (unsigned)g.n_px - blockIdx.x * TPX);  // pixels of this block
    const unsigned n = live ? px / (unsigned)g.hw : 0u;
    const unsigned r = live ? px - n * (unsigned)g.hw : 0u;
    if (warp == 0) {
        const unsigned h = r / (unsigned)g.iw, w = r - h * (unsigned)g.iw;
        const long row = g.lead + ((long)n * g.hp + h) * g.wp + w;
        row_s[lane] = live ? row * (g.words >> 1) : -1;
    }

    // channel extent walked: the channels, rounded up to whole 32-bit words of the packed row
    const int c_end = WITH_PACK ? min(g.words * 4, (g.ic + 3) & ~3) : g.ic;
    float acc = 0.f;
    // Warp w owns the TPER consecutive channels [TPER w, TPER (w + 1)) of every chunk.
    const int cw = TPER * warp;  // first channel of this warp inside a chunk
    const float *pw = g.src + (long)n * g.img_stride + r + (long)cw * g.hw;
    const unsigned pitch = (unsigned)g.hw * 4u;  // bytes between channels; the host checks the range
    float v[TPER];
    if (live && TCC <= g.ic) {
#pragma unroll
        for (int i = 0; i < TPER; i++) v[i] = ld_stream(row_ptr<TPER == 32>(pw, i, pitch));
    } else {
#pragma unroll
        for (int i = 0; i < TPER; i++)
            v[i] = (live && cw + i < g.ic) ? ld_stream(row_ptr<TPER == 32>(pw, i, pitch)) : 0.f;
    }
    for (int c0 = 0; c0 < c_end; c0 += TCC) {
        const bool full = c0 + TCC <= g.ic;  // no channel tail in this chunk
        if (WITH_A) {
            float4 *frow = reinterpret_cast<float4 *>(f_s + lane * FLD + cw);
#pragma unroll
            for (int j = 0; j < TPER / 4; j++)
                frow[j] = make_float4(__fmul_rn(fabsf(v[4 * j]), g.inv_ic),
                                      __fmul_rn(fabsf(v[4 * j + 1]), g.inv_ic),
                                      __fmul_rn(fabsf(v[4 * j + 2]), g.inv_ic),
                                      __fmul_rn(fabsf(v[4 * j + 3]), g.inv_ic));
        }
        if (WITH_PACK) {
            uint2 *brow = reinterpret_cast<uint2 *>(b_s + lane * TLD + cw);
#pragma unroll
            for (int j = 0; j < TPER / 8; j++) {
                uint32_t w2[2];
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int c = 8 * j + 4 * q;
                    uint32_t word = sign_bytes(v[c], v[c + 1], v[c + 2], v[c + 3]);
                    if (!full) {  // channels past the last one are zero bytes
                        const int left = g.ic - (c0 + cw + c);
                        word = left >= 4 ? word : left <= 0 ? 0u : (word & (0xFFFFFFFFu >> (8 * (4 - left))));
                    }
                    w2[q] = word;
                }
                brow[j] = make_uint2(w2[0], w2[1]);
            }
        }
        __syncthreads();
        if (c0 + TCC < c_end) {  // next chunk's loads fly while this one is consumed
            const float *pn = pw + (long)(c0 + TCC) * g.hw;
            if (live && c0 + 2 * TCC <= g.ic) {
#pragma unroll
                for (int i = 0; i < TPER; i++) v[i] = ld_stream(row_ptr<TPER == 32>(pn, i, pitch));
            } else {
#pragma unroll
                for (int i = 0; i < TPER; i++)
                    v[i] = (live && c0 + TCC + cw + i < g.ic) ? ld_stream(row_ptr<TPER == 32>(pn, i, pitch)) : 0.f;
            }
        }
        if (WITH_A && warp == 0) {
            const int nc = min(TCC, g.ic - c0);
            const float *fr = f_s + lane * FLD;
            if (nc == TCC) {
#pragma unroll
                for (int j0 = 0; j0 < TCC; j0 += 16) {
                    float4 t[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) t[j] = *reinterpret_cast<const float4 *>(fr + j0 + 4 * j);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        acc = __fadd_rn(acc, t[j].x);
                        acc = __fadd_rn(acc, t[j].y);
                        acc = __fadd_rn(acc, t[j].z);
                        acc = __fadd_rn(acc, t[j].w);
                    }
                }
            } else {  // channel tail: same order
                int j = 0;
                for (; j + 4 <= nc; j += 4) {
                    const float4 t = *reinterpret_cast<const float4 *>(fr + j);
                    acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, t.x), t.y), t.z), t.w);
                }
                for (; j < nc; j++) acc = __fadd_rn(acc, fr[j]);
            }
        } else if (WITH_PACK) {
            // half a warp writes one pixel per pass: 16 (12) lanes x 8 bytes, one 128-byte line
            const int first = WITH_A ? warp - 1 : warp, step = WITH_A ? TWARPS - 1 : TWARPS;
            const int n8 = (min(TCC, c_end - c0) + 7) / 8;
            constexpr int LPP = TCC / 8;   // lanes per pixel and chunk
            constexpr int PPW = 32 / LPP;  // pixels a warp writes per pass
            const int sub = lane / LPP, wl = lane % LPP;
            if (sub < PPW && wl < n8) {
                uint2 *out = reinterpret_cast<uint2 *>(g.out) + (c0 >> 3) + wl;
                const uint8_t *tile = b_s + 8 * wl;
                for (int pi = PPW * first + sub; pi < n_live; pi += PPW * step)
                    out[row_s[pi]] = *reinterpret_cast<const uint2 *>(tile + pi * TLD);
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

// tiled kernels: blocks per SM the carve-out is sized for (chunks of 128 and of 96 channels)
constexpr int kResidentBlocks = 5, kResidentBlocks96 = 9;

template <bool WITH_A, bool WITH_PACK>
cudaError_t launch_bin(const Plan &p, const BinArgs &g, cudaStream_t s) {
    const int threads = 128;
    const unsigned blocks = (unsigned)((g.n_px + threads - 1) / threads);
    if (blocks == 0) return cudaSuccess;
    if (!p.src_nhwc && (p.family == kTcgen05 || !WITH_PACK) && g.n_px < (1L << 31) - TPX &&
        (long)p.ih * p.iw < (1L << 24)) {
        // Shared-memory carve-out sized for a fixed number of blocks per SM, once per device. Left
        // to itself the driver sizes it for as many blocks as the thread count allows, which
        // leaves the L1 too small: the loads in flight occupy it although they do not allocate
        // lines to keep, and a kernel that streams with 32 loads per thread outstanding does not
        // need that many warps. Measured on conv4, minibatch 256, pass with the mean-|x| map:
        // eight blocks (an L1 of 32 KB) 20.4 us, seven or six (64 KB) 16.9-17.3, five (96 KB)
        // 17.0-17.1 with the whole step 0.5 us shorter, four or three (128 KB) 18.1. The
        // 96-channel kernel on conv2: nine of its blocks (the same 64 KB of L1) 9.3 us, seven
        // (96 KB) 9.7, five 11.2.
        static std::atomic<bool> tuned[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (!tuned[dev & 63].exchange(true, std::memory_order_acq_rel)) {
            int smem_sm = 0;
            cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
            auto carve = [&](auto kernel, int resident) {
                cudaFuncAttributes fa;
                if (smem_sm <= 0 || cudaFuncGetAttributes(&fa, kernel) != cudaSuccess) return;
                long pct = (100L * resident * ((long)fa.sharedSizeBytes + 1024) + smem_sm - 1) / smem_sm;
                if (pct > 100) pct = 100;
                cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)pct);
            };
            carve(binarize_bytes_nchw_kernel<WITH_A, WITH_PACK, 32>, kResidentBlocks);
            carve(binarize_bytes_nchw_kernel<WITH_A, WITH_PACK, 24>, kResidentBlocks96);
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
