// Launchers of the device kernels. Each takes the Plan, raw device pointers and a stream, and
// returns the CUDA status of the launch; none allocates or synchronises.
#pragma once

#include <atomic>

#include <cuda_runtime.h>

#include "plan.hpp"

namespace xb200 {

// Kernels launched by this library in this process (benchmark accounting).
extern std::atomic<long> g_kernel_launches;
inline void note_launch(int n = 1) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }

// Launch with programmatic stream serialisation: the grid may be scheduled while the previous
// kernel of the stream is still draining, so that its set-up (and the launch latency itself)
// runs under the predecessor's tail. Kernels launched this way call dependency_wait() before
// they touch anything an earlier kernel may have written or may still be reading. The
// tensor-core convolution and the tiled binarizer are launched like this (measured: 2-3 us per
// forward pass for the convolution, another 0.8 us for the binarizer in back-to-back passes).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t s, int cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cluster > 1) {  // thread-block clusters of `cluster` CTAs along x
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)cluster;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#ifdef __CUDACC__
// Lets the next kernel of the stream start its set-up now ...
__device__ __forceinline__ void dependency_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// ... and blocks until every earlier kernel of the stream has completed and its writes are
// visible. A no-op for grids launched the ordinary way.
__device__ __forceinline__ void dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

// ---- activations -----------------------------------------------------------------------------
// One pass over the fp32 source: sign bits into the family's packed layout and, when `a` is not
// null, the per-pixel mean |x| map. Replaces upstream src/bcast_binarize_data.cpp:43-73 and the
// first loop of src/bcast_calculate_k.cpp:49-66.
cudaError_t launch_binarize_data(const Plan &p, const float *src, void *bin_src, float *a,
                                 cudaStream_t s);
// The mean |x| map alone (calculate_k called on its own).
cudaError_t launch_mean_abs(const Plan &p, const float *src, float *a, cudaStream_t s);
// K = box filter of A over the filter window / (KH*KW), zero outside the image.
// Replaces the second loop of upstream src/bcast_calculate_k.cpp:69-85.
cudaError_t launch_box_filter(const Plan &p, const float *a, float *k, cudaStream_t s);

// ---- weights ---------------------------------------------------------------------------------
// Sign-pack into the family's layout, alpha[oc] = mean |w|, op_c[oh][ow] = IC * taps inside.
// Replaces upstream src/bcast_binarize_weights.cpp:54-142.
cudaError_t launch_binarize_weights(const Plan &p, const float *w, void *bin_w, float *alpha,
                                    int32_t *op_c, cudaStream_t s);

// to = sign(from) * mean(from) over `elems` device floats (upstream
// src/binarize_weights_float.cpp:3-25), with a fixed summation shape. Takes and returns a few
// hundred bytes of stream-ordered scratch.
cudaError_t launch_binarize_weights_float(long elems, const float *from, float *to,
                                          cudaStream_t s);

// ---- convolution -----------------------------------------------------------------------------
// dst = ((float)S * alpha) * K with S the signed agreement count over in-bounds taps
// (upstream src/default/bcast_convolution_default.cpp:60-103). When `sums` is not null the raw
// integers S are written there (NCHW int32) and dst is left alone.
cudaError_t launch_conv_popc(const Plan &p, const uint32_t *bin_src, const uint32_t *bin_w,
                             const float *alpha, const float *k, const int32_t *op_c, float *dst,
                             int32_t *sums, cudaStream_t s);

// The same contract on the tensor cores (tcgen05.mma kind::i8 over +-1 bytes, plan.hpp's framed
// layout). `error_word` is a device int the kernel sets non-zero if one of its bounded waits
// ran out; it is never cleared by the kernel. With k == nullptr the epilogue box-filters K from
// the mean-|x| map `a` itself (same arithmetic as launch_box_filter) and records it in k_out,
// which saves the separate stencil launch in the fused forward call.
//
// `next` chains two layers in the packed domain: instead of storing floats, the epilogue writes
// the sign of every result into the following layer's byte frame and the mean |result| over the
// filters into its mean-|x| map, which is what that layer's binarize_data and the first half of
// its calculate_k would have produced from the stored floats (upstream
// src/bcast_binarize_data.cpp:43-73, src/bcast_calculate_k.cpp:49-66). The signs are exact; the
// mean is summed per group of filters and folded in a fixed order, so it is reproducible but
// rounds differently from upstream's strictly sequential sum.
struct ChainTarget {
    void *bin_src;        // the next layer's res[bin_src]
    float *a;             // the next layer's res[a]
    int wp, hp, lead, icp;  // its frame geometry (Plan)
    float inv_ic;         // its Plan::inv_ic
};
// `test` (normally null) shortens a tensor-core kernel's wait limit and makes one CTA lose the
// commit that publishes its first accumulator, so that a test can watch a bounded wait run out:
// the kernel returns by itself with *error_word set and the results of the call invalid.
struct ConvSelfTest {
    unsigned long long wait_ns;  // 0: the normal limit (2 s)
    int drop_commit;
};
cudaError_t launch_conv_tcgen05(const Plan &p, const void *bin_src, const void *bin_w,
                                const float *alpha, const float *k, const float *a, float *k_out,
                                float *dst, int32_t *sums, int *error_word, cudaStream_t s,
                                const ChainTarget *next = nullptr,
                                const ConvSelfTest *test = nullptr);

// The same contract (without chaining) with the operand roles swapped: 128 filters on the UMMA M
// side, whole output rows of one image on the N side (Plan::img_*, conv_tcgen05_img.cu). Reads
// the same packed operands as launch_conv_tcgen05; the forward pass uses it when Plan::img is set.
cudaError_t launch_conv_tcgen05_img(const Plan &p, const void *bin_src, const void *bin_w,
                                    const float *alpha, const float *k, const float *a,
                                    float *k_out, float *dst, int32_t *sums, int *error_word,
                                    cudaStream_t s, const ConvSelfTest *test = nullptr);

}  // namespace xb200
