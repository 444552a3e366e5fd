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
        case kMmaB1: return "mma_b1";
        case kTcgen05: return "tcgen05_i8";
        default: return "auto";
    }
}

static Family family_from_env() {
    const char *e = getenv("XNOR_NN_B200_KERNEL");
    if (!e) return kAuto;
    if (!strcmp(e, "popc")) return kPopc;
    if (!strcmp(e, "mma_b1")) return kMmaB1;
    if (!strcmp(e, "tcgen05_i8") || !strcmp(e, "tcgen05")) return kTcgen05;
    return kAuto;
}

// The two tensor-core families walk a zero-framed image with constant row shifts per filter
// tap, which only describes a unit-stride convolution whose output extent matches the padding
// actually applied (upstream derives the output height from pw, src/common_convolution.cpp:16).
static bool frame_walk_ok(const Plan &p) {
    return p.sh == 1 && p.sw == 1 && p.oh == p.ih + 2 * p.ph - p.kh + 1 &&
           p.ow == p.iw + 2 * p.pw - p.kw + 1 && p.oh > 0 && p.ow > 0 &&
           p.kh - 1 - p.ph <= p.ph + p.ih && p.kw - 1 - p.pw <= p.iw &&
           (long)p.mb * (p.ih + p.ph) * (p.iw + p.pw) < (1L << 30);
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

    Family f = requested == kAuto ? family_from_env() : requested;
    const bool walk = frame_walk_ok(*p);
    if (f == kAuto) f = walk ? kTcgen05 : kPopc;
    // mma.sync b1 was measured and ruled out (its ceiling is below what the popc kernel
    // achieves); a request for it is served by popc.
    if (f == kMmaB1) f = kPopc;
    if (f == kTcgen05 && !walk) f = kPopc;
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

    if (f == kPopc) {
        p->ocp = div_up_i(p->oc, 8) * 8;
        p->bytes[xnor_nn_resource_bin_src] = px_in * p->icw * sizeof(uint32_t);
        p->bytes[xnor_nn_resource_bin_weights] =
            (size_t)p->kh * p->kw * p->icw * p->ocp * sizeof(uint32_t);
    } else {
        // K chunk = bytes of one channel group per pipeline stage = the swizzle span. Wide
        // chunks mean few, fat stages (4 MMAs per barrier round trip at 128 B), which is worth
        // some zero padding of the channels: 96 channels padded to 128 run the 5x5 AlexNet layer
        // in 67 us, as three 32-byte chunks in 89 us. Take the widest chunk that pads the
        // channels by no more than 35 %.
        p->kchunk = 32;
        for (int k = 128; k >= 64; k /= 2)
            if (div_up_i(p->ic, k) * k <= p->ic * 1.35) { p->kchunk = k; break; }
        if (const char *e = getenv("XNOR_NN_B200_KCHUNK")) {  // tuning override: 32, 64 or 128
            const int v = atoi(e);
            if (v == 32 || v == 64 || v == 128) p->kchunk = v;
        }
        p->icp = div_up_i(p->ic, p->kchunk) * p->kchunk;
        // Filter tile = UMMA N: a multiple of 16, at most 256. The filters are split into the
        // fewest equal tiles and padded (with zero filters) to fill them, so N stays as wide as
        // possible: the kernel is bound by the instruction stream that issues the MMAs, whose
        // cost per instruction does not shrink with N (conv4 on 128 images: 32.9 us at N=128
        // against 26.7 us at N=256).
        // Exception: when the whole layer is fewer tiles than half the SMs (small minibatches,
        // e.g. one GPU's share of a sharded batch), halving N doubles the SMs at work without
        // adding a round of tiles; below N=128 the per-instruction cost eats the gain.
        const int fewest = div_up_i(p->oc, 256);
        int n_tiles = fewest;
        const long m_tiles = (p->q_total + 127) / 128;
        while (m_tiles * n_tiles * 2 <= sm_count() && div_up_i(p->oc, n_tiles * 2) >= 128)
            n_tiles *= 2;
        if (const char *e = getenv("XNOR_NN_B200_NTILES")) {  // tuning override
            const int v = atoi(e);
            if (v >= fewest && div_up_i(p->oc, v) >= 16) n_tiles = v;
        }
        p->n_tile = div_up_i(div_up_i(p->oc, n_tiles), 16) * 16;
        p->ocp16 = p->n_tile * n_tiles;
        p->lead = p->ph * p->wp + p->pw;
        p->rows = p->lead + p->q_total + 256 + (long)p->kh * p->wp + p->kw;
        p->bytes[xnor_nn_resource_bin_src] = (size_t)p->rows * p->icp;
        p->bytes[xnor_nn_resource_bin_weights] = (size_t)p->kh * p->kw * p->ocp16 * p->icp;
    }
}

}  // namespace xb200
