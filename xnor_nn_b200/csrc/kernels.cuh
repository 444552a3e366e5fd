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
cudaError_t launch_conv_tcgen05(const Plan &p, const void *bin_src, const void *bin_w,
                                const float *alpha, const float *k, const float *a, float *k_out,
                                float *dst, int32_t *sums, int *error_word, cudaStream_t s);

}  // namespace xb200
