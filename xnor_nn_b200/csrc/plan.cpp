#include "plan.hpp"

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

namespace xb200 {

// SMs of the current device (148 on B200); the same figure when no device can be asked, so that
// plans made on a machine without a GPU come out as they would on the target.
static int sm_count() {
    static const int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
            (void)cudaGetLastError();
            v = 148;
        }
        return v;
    }();
    return n;
}

int div_up_i(int a, int b) { return (a + b - 1) / b; }

const char *family_name(Family f) {
    switch (f) {
        case kPopc: return "popc";
        case kTcgen05: return "tcgen05_i8";
        case kTcgen05Rows: return "tcgen05_i8_rows";
        default: return "auto";
    }
}

static Family family_from_env() {
    const char *e = getenv("XNOR_NN_B200_KERNEL");
    if (!e) return kAuto;
    if (!strcmp(e, "popc")) return kPopc;
    if (!strcmp(e, "tcgen05_i8") || !strcmp(e, "tcgen05")) return kTcgen05;
    if (!strcmp(e, "tcgen05_i8_rows")) return kTcgen05Rows;
    return kAuto;
}

// Both tensor-core kernels read the zero-framed activation bytes and describe a unit-stride
// convolution only.
static bool unit_stride(const Plan &p) {
    return p.sh == 1 && p.sw == 1 && p.oh > 0 && p.ow > 0 &&
           (long)p.mb * (p.ih + p.ph) * (p.iw + p.pw) < (1L << 30);
}

// The position-tile kernel walks the frame with one constant row shift per filter tap. That
// needs the output extent to match the padding actually applied (upstream derives the output
// height from pw, src/common_convolution.cpp:16) and every output pixel to have a frame position
// of its own, i.e. a padding smaller than the filter (with ph >= kh the output has more rows
// than the frame).
static bool frame_walk_ok(const Plan &p) {
    return unit_stride(p) && p.oh == p.ih + 2 * p.ph - p.kh + 1 &&
           p.ow == p.iw + 2 * p.pw - p.kw + 1 && p.ph < p.kh && p.pw < p.kw &&
           p.kh - 1 - p.ph <= p.ph + p.ih && p.kw - 1 - p.pw <= p.iw;
}

// The image-row kernel addresses the frame as a 4-D tensor (channel, column, row, image) and lets
// the copy engine fill whatever lies outside with zeros, so any padding and any output extent
// work; a tile must hold at least one whole output row.
static bool image_rows_ok(const Plan &p) { return unit_stride(p) && p.ow <= 256; }

// Relative duration of a tile whose UMMA N is n: an instruction occupies the tensor pipe for n/2
// cycles, but the issuing thread needs about 45 cycles per tcgen05.mma and 275 per
// tcgen05.commit (measured); with a commit after every four instructions that is 113 cycles per
// instruction, which is what an N of 226 takes.
static long tile_cost(int n) { return n < 226 ? 226 : n; }

int img_staging_row_words(const Plan &p) {
    int w = (p.img_rows * p.ow + 3 + 3) & ~3;
    if (w % 8 == 0) w += 4;  // an odd multiple of 4: eight rows before a bank repeats
    return w;
}

size_t img_staging_bytes(const Plan &p) {
    size_t words = 32 * (size_t)img_staging_row_words(p);
    if (p.img_row_blocks == 1 && 32 * (size_t)p.oh * p.ow > words) words = 32 * (size_t)p.oh * p.ow;
    return (words * 4 + 127) & ~(size_t)127;
}

void plan_image_rows(Plan *p) {
    p->img = false;
    if (p->family != kTcgen05 || !p->img_forced || !image_rows_ok(*p) || p->mb < 1) return;
    const int sms = sm_count();
    const int m_blocks = div_up_i(p->oc, 128);
    long best = -1;
    int best_r = 0;
    for (int r = 1; r <= p->oh && r * p->ow <= 256; r++) {
        const int n = div_up_i(r * p->ow, 16) * 16;
        const long tiles = (long)p->mb * div_up_i(p->oh, r) * m_blocks;
        const long rem = tiles % sms;
        long cost = (tiles / sms) * tile_cost(n);
        if (rem) {
            const long half = tile_cost(div_up_i((r + 1) / 2 * p->ow, 16) * 16);
            const bool split = r >= 2 && 2 * rem <= sms && half < tile_cost(n);
            cost += split ? half : tile_cost(n);
        }
        if (best < 0 || cost <= best) { best = cost; best_r = r; }  // ties: the larger tile
    }
    const int r = best_r;
    p->img_rows = r;
    p->img_n = div_up_i(r * p->ow, 16) * 16;
    p->img_row_blocks = div_up_i(p->oh, r);
    p->img_m_blocks = m_blocks;
    const long tiles = (long)p->mb * p->img_row_blocks * m_blocks;
    if (tiles >= (1L << 30)) return;
    p->img_tiles = (int)tiles;
    const int rem = (int)(tiles % sms);
    const bool split = rem && r >= 2 && 2 * rem <= sms &&
                       tile_cost(div_up_i((r + 1) / 2 * p->ow, 16) * 16) < tile_cost(p->img_n);
    p->img_whole = split ? (int)tiles - rem : (int)tiles;
    p->img_half_rows = split ? (r + 1) / 2 : 0;
    p->img_n_half = split ? div_up_i(p->img_half_rows * p->ow, 16) * 16 : 0;
    const long units = (long)p->img_whole + 2L * (tiles - p->img_whole);
    p->img_grid = (int)(units < sms ? units : sms);

    // Shared memory: control block, operand ring, result staging. Two staging buffers let one
    // pair of epilogue warps fill while the other pair's bulk stores drain; a deep operand ring
    // matters more, so staging shrinks first.
    const long stage = ((long)(128 + p->img_n) * p->kchunk + 1023) & ~1023L;
    const long staging = (long)img_staging_bytes(*p);
    const long budget = 227 * 1024 - 1024 - 2304;  // alignment slack, control block
    int n_staging = 2;
    long stages = (budget - n_staging * staging) / stage;
    if (stages < 4) {
        n_staging = 1;
        stages = (budget - staging) / stage;
    }
    if (stages < 2) return;
    p->img_stages = (int)(stages > 8 ? 8 : stages);
    p->img_staging = n_staging;

    p->img = true;
}

void make_plan(Plan *p, const xnor_nn_convolution_t *c, Family requested) {
    memset(p, 0, sizeof(*p));
    p->mb = c->mb; p->ic = c->ic; p->ih = c->ih; p->iw = c->iw;
    p->oc = c->oc; p->oh = c->oh; p->ow = c->ow;
    p->kh = c->kh; p->kw = c->kw; p->sh = c->sh; p->sw = c->sw; p->ph = c->ph; p->pw = c->pw;
    p->src_nhwc = c->src_format == xnor_nn_data_format_nhwc;
    p->w_hwio = c->weights_format == xnor_nn_weights_format_hwio;
    p->dst_nhwc = c->dst_format == xnor_nn_data_format_nhwc;
    p->formats_ok =
        (c->src_format == xnor_nn_data_format_nchw || c->src_format == xnor_nn_data_format_nhwc) &&
        (c->weights_format == xnor_nn_weights_format_oihw ||
         c->weights_format == xnor_nn_weights_format_hwio) &&
        (c->dst_format == xnor_nn_data_format_nchw || c->dst_format == xnor_nn_data_format_nhwc);

    p->inv_ic = 1.f / p->ic;
    p->inv_khw = 1.f / p->kh / p->kw;
    p->inv_chw = 1.f / (p->ic * p->kh * p->kw);

    // The position-tile kernel serves every shape it can: with one tcgen05.commit per four
    // instructions a tile costs the same whatever its N, so the shape with the fewest tiles wins,
    // and that kernel's tiles are always 128 x 256 (measured on the five benchmark layers: 36 /
    // 44 / 68 / 95 us against 45 / 49 / 74 / 109 us). The image-row kernel takes what is left:
    // paddings as large as the filter, output extents that do not follow from the padding.
    Family f = requested;
    if (f != kPopc && f != kTcgen05 && f != kTcgen05Rows) f = family_from_env();
    const bool frame = frame_walk_ok(*p), rows = image_rows_ok(*p);
    if (f == kAuto) f = (frame || rows) ? kTcgen05 : kPopc;
    const bool force_rows = f == kTcgen05Rows;
    if (force_rows) f = rows ? kTcgen05 : kPopc;
    if (f == kTcgen05 && !frame && !rows) f = kPopc;
    p->family = f;

    const size_t px_in = (size_t)p->mb * p->ih * p->iw;
    const size_t px_out = (size_t)p->mb * p->oh * p->ow;
    p->bytes[xnor_nn_resource_alpha] = (size_t)p->oc * sizeof(float);
    p->bytes[xnor_nn_resource_a] = px_in * sizeof(float);
    p->bytes[xnor_nn_resource_k] = px_out * sizeof(float);
    p->bytes[xnor_nn_resource_operations_count] = (size_t)p->oh * p->ow * sizeof(int32_t);

    p->icw = div_up_i(p->ic, 32);
    p->wp = p->iw + p->pw;
    p->hp = p->ih + p->ph;
    p->q_total = (long)p->mb * p->hp * p->wp;

    auto plan_popc = [&] {
        p->family = kPopc;
        p->img = false;
        p->ocp = div_up_i(p->oc, 8) * 8;
        p->bytes[xnor_nn_resource_bin_src] = px_in * p->icw * sizeof(uint32_t);
        p->bytes[xnor_nn_resource_bin_weights] =
            (size_t)p->kh * p->kw * p->icw * p->ocp * sizeof(uint32_t);
    };
    if (f == kPopc) {
        plan_popc();
        return;
    }
    // K chunk = bytes of one channel group per pipeline stage = the swizzle span. Wide chunks
    // mean few, fat stages (4 MMAs per barrier round trip at 128 B), which is worth some zero
    // padding of the channels: 96 channels padded to 128 run the 5x5 AlexNet layer in 67 us, as
    // three 32-byte chunks in 89 us. Take the widest chunk that pads the channels by no more
    // than 35 %.
    p->kchunk = 32;
    for (int k = 128; k >= 64; k /= 2)
        if (div_up_i(p->ic, k) * k <= p->ic * 1.35) { p->kchunk = k; break; }
    p->icp = div_up_i(p->ic, p->kchunk) * p->kchunk;
    // Filter tile of the position-tile kernel = its UMMA N: a multiple of 16, at most 256. The
    // filters are split into the fewest equal tiles and padded (with zero filters) to fill them,
    // so N stays as wide as possible: the kernel is bound by the instruction stream that issues
    // the MMAs, whose cost per instruction does not shrink with N. When the whole layer is fewer
    // tiles than half the SMs, halving N doubles the SMs at work without adding a round of
    // tiles; below N=128 the per-instruction cost eats the gain.
    // The same number is the row count of a filter tap in the packed weight matrix, which both
    // tensor-core kernels read.
    const int fewest = div_up_i(p->oc, 256);
    int n_tiles = fewest;
    const long m_tiles = (p->q_total + 127) / 128;
    while (m_tiles * n_tiles * 2 <= sm_count() && div_up_i(p->oc, n_tiles * 2) >= 128)
        n_tiles *= 2;
    p->n_tile = div_up_i(div_up_i(p->oc, n_tiles), 16) * 16;
    p->ocp16 = p->n_tile * n_tiles;
    p->lead = p->ph * p->wp + p->pw;
    p->rows = p->lead + p->q_total + 256 + (long)p->kh * p->wp + p->kw;
    p->bytes[xnor_nn_resource_bin_src] = (size_t)p->rows * p->icp;
    p->bytes[xnor_nn_resource_bin_weights] = (size_t)p->kh * p->kw * p->ocp16 * p->icp;
    p->img_forced = force_rows || !frame;
    plan_image_rows(p);
    if (!p->img && !frame) plan_popc();  // neither tensor-core kernel can serve the shape
}

}  // namespace xb200
