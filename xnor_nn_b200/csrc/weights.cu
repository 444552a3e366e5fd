// Weight-side kernels: sign packing, alpha = mean |w| per output channel, and the per-pixel
// count of contributing operands. They run once per weight change (a few hundred KB of
// output), off the per-minibatch path, so they favour exactness over speed: alpha is summed by
// one thread per output channel in upstream's (ic, kh, kw) order
// (src/bcast_binarize_weights.cpp:99-114) and therefore rounds identically.
#include "kernels.cuh"

namespace xb200 {

namespace {

struct WArgs {
    const float *w;
    int oc, ic, kh, kw;
    bool hwio;
};

__device__ __forceinline__ long w_index(const WArgs &g, int oc, int c, int kh, int kw) {
    return g.hwio ? (((long)kh * g.kw + kw) * g.ic + c) * g.oc + oc
                  : (((long)oc * g.ic + c) * g.kh + kh) * g.kw + kw;
}

__device__ __forceinline__ unsigned sign_clear(float x) { return (~__float_as_uint(x)) >> 31; }

// bits: uint32 [tap][word][ocp]
__global__ void pack_weight_bits_kernel(const WArgs g, uint32_t *out, int icw, int ocp) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long total = (long)g.kh * g.kw * icw * ocp;
    if (i >= total) return;
    const int oc = (int)(i % ocp);
    const int word = (int)((i / ocp) % icw);
    const int tap = (int)(i / ((long)ocp * icw));
    const int kh = tap / g.kw, kw = tap - kh * g.kw;
    uint32_t v = 0;
    for (int b = 0; b < 32; b++) {
        const int c = word * 32 + b;
        unsigned bit = 0;
        if (oc < g.oc && c < g.ic) bit = sign_clear(__ldg(g.w + w_index(g, oc, c, kh, kw)));
        v = (v << 1) | bit;
    }
    out[i] = v;
}

// bytes: int8 [tap][ocp16][icp], +1 / -1, zero where the channel or the filter does not exist
__global__ void pack_weight_bytes_kernel(const WArgs g, uint32_t *out, int icp, int ocp16) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int groups = icp / 4;
    const long total = (long)g.kh * g.kw * ocp16 * groups;
    if (i >= total) return;
    const int grp = (int)(i % groups);
    const int oc = (int)((i / groups) % ocp16);
    const int tap = (int)(i / ((long)groups * ocp16));
    const int kh = tap / g.kw, kw = tap - kh * g.kw;
    uint32_t v = 0;
    for (int b = 0; b < 4; b++) {
        const int c = grp * 4 + b;
        if (oc < g.oc && c < g.ic)
            v |= (sign_clear(__ldg(g.w + w_index(g, oc, c, kh, kw))) ? 0x01u : 0xFFu) << (8 * b);
    }
    out[i] = v;
}

// alpha[oc] = sum over (ic, kh, kw) ascending of |w| * (1/(IC*KH*KW)), one thread per filter so
// that the additions happen in upstream's order. A block owns 32 filters; the weights are staged
// through shared memory in chunks so that the global reads are coalesced (OIHW: each filter's
// weights are one contiguous run; HWIO: 32 neighbouring filters are contiguous for each (tap, ic)).
constexpr int ACH = 128;  // elements of the (ic, kh, kw) walk per chunk

__global__ void __launch_bounds__(256) alpha_kernel(const WArgs g, float *alpha, float inv_chw) {
    __shared__ float t[32][ACH + 1];
    const int oc0 = blockIdx.x * 32;
    const int n = g.ic * g.kh * g.kw, khw = g.kh * g.kw;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float acc = 0.f;
    for (int e0 = 0; e0 < n; e0 += ACH) {
        const int ne = min(ACH, n - e0);
        if (!g.hwio) {
            // warp w stages filters w, w+8, ...: lanes walk the contiguous run of one filter
            for (int f = warp; f < 32; f += 8)
                for (int e = lane; e < ne; e += 32)
                    t[f][e] = oc0 + f < g.oc ? fabsf(__ldg(g.w + (long)(oc0 + f) * n + e0 + e)) : 0.f;
        } else {
            // lanes walk 32 neighbouring filters of one (ic, kh, kw) element
            for (int e = warp; e < ne; e += 8) {
                const int idx = e0 + e;  // position in upstream's (ic, kh, kw) walk
                const int c = idx / khw, tap = idx - c * khw;
                t[lane][e] = oc0 + lane < g.oc
                                 ? fabsf(__ldg(g.w + ((long)tap * g.ic + c) * g.oc + oc0 + lane))
                                 : 0.f;
            }
        }
        __syncthreads();
        if (warp == 0)
            for (int e = 0; e < ne; e++) acc = __fadd_rn(acc, __fmul_rn(t[lane][e], inv_chw));
        __syncthreads();
    }
    if (warp == 0 && oc0 + lane < g.oc) alpha[oc0 + lane] = acc;
}

__global__ void op_count_kernel(int32_t *op_c, int ic, int ih, int iw, int oh, int ow, int kh,
                                int kw, int sh, int sw, int ph, int pw) {
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= oh * ow) return;
    const int y = o / ow, x = o - y * ow;
    int taps = 0;
    for (int i = 0; i < kh; i++) {
        const int h = y * sh - ph + i;
        if (h < 0 || h >= ih) continue;
        for (int j = 0; j < kw; j++) {
            const int w = x * sw - pw + j;
            taps += (w >= 0 && w < iw);
        }
    }
    op_c[o] = taps * ic;
}

}  // namespace

cudaError_t launch_binarize_weights(const Plan &p, const float *w, void *bin_w, float *alpha,
                                    int32_t *op_c, cudaStream_t s) {
    WArgs g;
    g.w = w; g.oc = p.oc; g.ic = p.ic; g.kh = p.kh; g.kw = p.kw; g.hwio = p.w_hwio;
    const int threads = 128;
    if (p.family == kTcgen05) {
        const long total = (long)p.kh * p.kw * p.ocp16 * (p.icp / 4);
        pack_weight_bytes_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, s>>>(
            g, (uint32_t *)bin_w, p.icp, p.ocp16);
    } else {
        const long total = (long)p.kh * p.kw * p.icw * p.ocp;
        pack_weight_bits_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, s>>>(
            g, (uint32_t *)bin_w, p.icw, p.ocp);
    }
    note_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    alpha_kernel<<<(p.oc + 31) / 32, 256, 0, s>>>(g, alpha, p.inv_chw);
    note_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    op_count_kernel<<<(p.oh * p.ow + threads - 1) / threads, threads, 0, s>>>(
        op_c, p.ic, p.ih, p.iw, p.oh, p.ow, p.kh, p.kw, p.sh, p.sw, p.ph, p.pw);
    note_launch();
    return cudaGetLastError();
}

// ---- float binarisation for the training backward pass ----------------------------------------
// to = sign(from) * mean(from) over the whole filter bank (upstream
// src/binarize_weights_float.cpp:3-25; the mean is of the signed values, as upstream has it).
// Upstream accumulates the sum in an OpenMP loop without a reduction clause, so its result depends
// on the thread schedule; here the sum has one fixed shape: thread t of block b adds elements
// b*256 + t, + 65536, + 131072, ... in ascending order, a block folds its 256 running sums with
// a fixed binary tree, and every block of the second kernel folds the 256 block sums with the
// same tree. The result is therefore reproducible and within rounding of the one-thread sum.
namespace {
constexpr int kWfBlocks = 256, kWfThreads = 256;

__device__ __forceinline__ float fold256(float v, float *sh) {
    sh[threadIdx.x] = v;
    __syncthreads();
    for (int w = kWfThreads / 2; w > 0; w >>= 1) {
        if ((int)threadIdx.x < w) sh[threadIdx.x] = __fadd_rn(sh[threadIdx.x], sh[threadIdx.x + w]);
        __syncthreads();
    }
    return sh[0];
}

__global__ void __launch_bounds__(kWfThreads) wf_partial_kernel(const float *from, long elems,
                                                                float *partial) {
    __shared__ float sh[kWfThreads];
    float acc = 0.f;
    for (long i = (long)blockIdx.x * kWfThreads + threadIdx.x; i < elems;
         i += (long)kWfBlocks * kWfThreads)
        acc = __fadd_rn(acc, from[i]);
    const float total = fold256(acc, sh);
    if (threadIdx.x == 0) partial[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kWfThreads) wf_scale_kernel(const float *from, float *to,
                                                              long elems, const float *partial,
                                                              float inv_elems) {
    __shared__ float sh[kWfThreads];
    const float mean = __fmul_rn(fold256(partial[threadIdx.x], sh), inv_elems);
    for (long i = (long)blockIdx.x * kWfThreads + threadIdx.x; i < elems;
         i += (long)gridDim.x * kWfThreads)
        to[i] = __fmul_rn(from[i] >= .0f ? 1.f : -1.f, mean);
}
}  // namespace

cudaError_t launch_binarize_weights_float(long elems, const float *from, float *to,
                                          cudaStream_t s) {
    float *partial = nullptr;
    cudaError_t e = cudaMallocAsync(&partial, kWfBlocks * sizeof(float), s);
    if (e != cudaSuccess) return e;
    wf_partial_kernel<<<kWfBlocks, kWfThreads, 0, s>>>(from, elems, partial);
    note_launch();
    long blocks = (elems + kWfThreads - 1) / kWfThreads;
    if (blocks > 1184) blocks = 1184;
    if (blocks < 1) blocks = 1;
    wf_scale_kernel<<<(unsigned)blocks, kWfThreads, 0, s>>>(from, to, elems, partial,
                                                            1.f / (float)elems);
    note_launch();
    e = cudaGetLastError();
    const cudaError_t f = cudaFreeAsync(partial, s);
    return e != cudaSuccess ? e : f;
}

}  // namespace xb200
