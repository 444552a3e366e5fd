// Direct XNOR/popcount convolution on the integer pipe (LOP3 + POPC + IADD).
//
// This is the general kernel: any stride, padding, filter size and tensor format, no
// restriction on the number of output channels. A block owns 128 output pixels x 64 output
// channels; a warp owns 8 of the channels, a lane 4 neighbouring pixels, 32 accumulators per
// thread. For each filter tap the block stages the packed activations of its 128 pixels in
// shared memory (word-major, so a lane fetches its 4 pixels with one 16-byte load) together
// with an all-ones / all-zero word per pixel that says whether the tap falls inside the image;
// out-of-image taps are thereby skipped, as upstream skips them
// (src/default/bcast_convolution_default.cpp:71-72). Weight words are the same for every lane
// of a warp and arrive as broadcast 16-byte loads through L1.
//
// With D = sum over in-bounds taps of popcount(a xor w) (absent channels are 0 on both sides),
// the signed agreement count is S = op_c - 2*D, op_c = IC * in-bounds taps, which equals
// upstream's 2*popcount(xnor) - op_c.
//
// Bound: the POPC issue rate (a quarter of the LOP3/IADD rate), see the roofline notes of the
// benchmark; the packed operands total a few MB and stay in L2.
#include "kernels.cuh"

namespace xb200 {

namespace {

constexpr int TM = 128;       // pixels per block
constexpr int TN = 64;        // output channels per block
constexpr int WCH = 16;       // words of K staged per step
constexpr int LDA = TM + 4;   // padded row of the staged tile, keeps 16-byte alignment

struct ConvArgs {
    const uint32_t *a;
    const uint32_t *w;
    const float *alpha;
    const float *k;
    const int32_t *op_c;
    float *dst;
    int32_t *sums;
    long m_total;  // mb*oh*ow
    int ih, iw, oc, oh, ow, kh, kw, sh, sw, ph, pw;
    int icw, ocp;
    bool dst_nhwc;
};

__global__ void __launch_bounds__(256) conv_popc_kernel(const ConvArgs g) {
    __shared__ __align__(16) uint32_t a_s[WCH * LDA];
    __shared__ __align__(16) uint32_t mask_s[TM];
    __shared__ int px_n[TM], px_r[TM], px_h0[TM], px_w0[TM];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long m0 = (long)blockIdx.x * TM;
    const int n0 = blockIdx.y * TN + warp * 8;
    const int ohw = g.oh * g.ow;

    if (tid < TM) {
        const long m = m0 + tid;
        if (m < g.m_total) {
            const int n = (int)(m / ohw);
            const int r = (int)(m - (long)n * ohw);
            const int oh = r / g.ow, ow = r - oh * g.ow;
            px_n[tid] = n; px_r[tid] = r;
            px_h0[tid] = oh * g.sh - g.ph; px_w0[tid] = ow * g.sw - g.pw;
        } else {
            px_n[tid] = -1; px_r[tid] = 0; px_h0[tid] = 0; px_w0[tid] = 0;
        }
    }

    int acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0;

    const bool warp_active = n0 < g.ocp;  // whole warp past the padded channel range idles

    for (int kh = 0; kh < g.kh; kh++)
        for (int kw = 0; kw < g.kw; kw++) {
            const int tap = kh * g.kw + kw;
            for (int wc = 0; wc < g.icw; wc += WCH) {
                const int nw = min(WCH, g.icw - wc);
                __syncthreads();  // previous step's readers are done (and px_* are visible)
                for (int i = tid; i < TM * nw; i += 256) {
                    const int px = i / nw, word = i - px * nw;
                    const int ih = px_h0[px] + kh, iw = px_w0[px] + kw;
                    const bool in = px_n[px] >= 0 && ih >= 0 && ih < g.ih && iw >= 0 && iw < g.iw;
                    uint32_t v = 0;
                    if (in)
                        v = __ldg(g.a + (((long)px_n[px] * g.ih + ih) * g.iw + iw) * g.icw + wc + word);
                    a_s[word * LDA + px] = v;
                    if (word == 0) mask_s[px] = in ? 0xffffffffu : 0u;
                }
                __syncthreads();
                if (warp_active) {
                    const uint4 m4 = *reinterpret_cast<const uint4 *>(&mask_s[4 * lane]);
                    const uint32_t mk[4] = {m4.x, m4.y, m4.z, m4.w};
                    const uint32_t *wrow = g.w + ((long)tap * g.icw + wc) * g.ocp + n0;
#pragma unroll 2
                    for (int word = 0; word < nw; word++) {
                        const uint4 a4 = *reinterpret_cast<const uint4 *>(&a_s[word * LDA + 4 * lane]);
                        const uint4 w0 = __ldg(reinterpret_cast<const uint4 *>(wrow + (long)word * g.ocp));
                        const uint4 w1 = __ldg(reinterpret_cast<const uint4 *>(wrow + (long)word * g.ocp + 4));
                        const uint32_t av[4] = {a4.x, a4.y, a4.z, a4.w};
                        const uint32_t wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                        for (int i = 0; i < 4; i++)
#pragma unroll
                            for (int j = 0; j < 8; j++)
                                acc[i][j] += __popc((av[i] ^ wv[j]) & mk[i]);
                    }
                }
            }
        }

    if (!warp_active) return;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int px = 4 * lane + i;
        const int n = px_n[px];
        if (n < 0) continue;
        const int r = px_r[px];
        const int opc = __ldg(g.op_c + r);
        const float kk = g.sums ? 0.f : __ldg(g.k + (long)n * ohw + r);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int oc = n0 + j;
            if (oc >= g.oc) break;
            const int s = opc - 2 * acc[i][j];
            if (g.sums) {
                g.sums[((long)n * g.oc + oc) * ohw + r] = s;
            } else {
                const float v = __fmul_rn(__fmul_rn((float)s, __ldg(g.alpha + oc)), kk);
                const long at = g.dst_nhwc ? ((long)n * ohw + r) * g.oc + oc
                                           : ((long)n * g.oc + oc) * ohw + r;
                g.dst[at] = v;
            }
        }
    }
}

}  // namespace

cudaError_t launch_conv_popc(const Plan &p, const uint32_t *bin_src, const uint32_t *bin_w,
                             const float *alpha, const float *k, const int32_t *op_c, float *dst,
                             int32_t *sums, cudaStream_t s) {
    ConvArgs g;
    g.a = bin_src; g.w = bin_w; g.alpha = alpha; g.k = k; g.op_c = op_c; g.dst = dst; g.sums = sums;
    g.m_total = (long)p.mb * p.oh * p.ow;
    g.ih = p.ih; g.iw = p.iw; g.oc = p.oc; g.oh = p.oh; g.ow = p.ow; g.kh = p.kh; g.kw = p.kw;
    g.sh = p.sh; g.sw = p.sw; g.ph = p.ph; g.pw = p.pw;
    g.icw = p.icw; g.ocp = p.ocp; g.dst_nhwc = p.dst_nhwc;
    if (g.m_total == 0) return cudaSuccess;
    dim3 grid((unsigned)((g.m_total + TM - 1) / TM), (unsigned)((p.oc + TN - 1) / TN));
    conv_popc_kernel<<<grid, 256, 0, s>>>(g);
    note_launch();
    return cudaGetLastError();
}

}  // namespace xb200
