/*
 * Entry points this library adds next to the upstream xnor_nn interface. None of them changes
 * the six upstream signatures in xnor_nn.h; a program that never includes this header behaves
 * exactly as it would against upstream, only on the GPU.
 *
 * Each declaration names the upstream code whose role it takes over, where there is one.
 */
#ifndef XNOR_NN_B200_H
#define XNOR_NN_B200_H

#include <stdint.h>

#include "xnor_nn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Kernel that consumes the packed operands. Upstream picks between its int16 and int32 word
 * paths and its per-ISA kernels inside xnor_nn_init_convolution (src/implementation.cpp:16-24,
 * src/bcast_convolution.cpp:92-117); this is the same decision for the GPU. `auto` honours the
 * environment variable XNOR_NN_B200_KERNEL (popc | tcgen05_i8 | tcgen05_i8_rows) and otherwise
 * picks by shape. Both tcgen05 kernels read the same packed operands (+-1 bytes), so chained
 * layers and single executors work with either.
 * (The value 1 is not used: the mma.sync b1 path it once named was measured slower than the
 * integer pipe and never built; a request for an unknown value is treated as `auto`.) */
typedef enum {
    xnor_nn_b200_kernel_auto = -1,
    xnor_nn_b200_kernel_popc = 0,            /* LOP3+POPC integer pipe; every shape and format */
    xnor_nn_b200_kernel_tcgen05_i8 = 2,      /* tcgen05.mma kind::i8, tiles of 128 frame
                                                positions x up to 256 filters; unit stride,
                                                padding smaller than the filter. Shapes it cannot
                                                serve go to the rows kernel, then to popc. */
    xnor_nn_b200_kernel_tcgen05_i8_rows = 3  /* tcgen05.mma kind::i8, tiles of 128 filters x
                                                whole output rows of one image; unit stride,
                                                rows of at most 256 pixels, any padding */
} xnor_nn_b200_kernel_t;

/* xnor_nn_init_convolution (src/common_convolution.cpp:9-63) with the kernel family stated.
 * A family that cannot serve the shape (strided convolutions on the tensor-core families)
 * degrades to popc, the way an upstream bcast request degrades to the reference algorithm
 * when oc is not a multiple of the vector width (src/bcast_convolution.cpp:45-56). */
xnor_nn_status_t xnor_nn_b200_init_convolution(xnor_nn_convolution_t *c,
                                               const xnor_nn_algorithm_t algorithm,
                                               const xnor_nn_tensor_format_t src_fmt,
                                               const xnor_nn_tensor_format_t weights_fmt,
                                               const xnor_nn_tensor_format_t dst_fmt,
                                               int mb, int oc, int ic, int ih, int iw,
                                               int kh, int kw, int sh, int sw, int ph, int pw,
                                               xnor_nn_b200_kernel_t kernel);

/* The family the descriptor ended up with. */
xnor_nn_b200_kernel_t xnor_nn_b200_kernel_of(const xnor_nn_convolution_t *c);

/* One call for what xnor_nn::Convolution::forward does with three (include/xnor_nn.hpp:45-53):
 * binarize_data, calculate_k and forward on res[user_src] -> res[user_dst]. The source crosses
 * to the device once instead of twice, and the mean-|x| map is produced by the packing pass. */
xnor_nn_status_t xnor_nn_b200_forward(const xnor_nn_convolution_t *c, xnor_nn_resources_t res);

/* The first of the two kernels xnor_nn_b200_forward runs, on its own: one pass over
 * res[user_src] that packs the signs into res[bin_src] (binarize_data,
 * src/bcast_binarize_data.cpp:43-73) and leaves the mean-|x| map in res[a] (the first loop of
 * calculate_k, src/bcast_calculate_k.cpp:49-66). For callers that want to overlap the packing of
 * one minibatch with other work, and for the benchmark, which times this kernel separately. */
xnor_nn_status_t xnor_nn_b200_binarize(const xnor_nn_convolution_t *c, xnor_nn_resources_t res);

/* Consecutive binary convolutions with no float tensor between them: layer i's results never
 * leave the chip as floats; the convolution kernel writes their signs straight into layer i+1's
 * packed input and their mean magnitude into its mean-|x| map, which is what layer i+1's
 * binarize_data and calculate_k (src/bcast_binarize_data.cpp:43-73,
 * src/bcast_calculate_k.cpp:49-66) would have derived from the stored floats. Upstream has no
 * such call; it stands for what its Caffe model does with conv3 -> conv4 -> conv5
 * (external/caffe/models/xnor_nn_alexnet/time.prototxt) minus the activation layers between them.
 *   c[i], res[i]: the layers in order, each initialised, allocated and with binarize_weights done;
 *   source: res[0][user_src]; result: res[layers-1][user_dst] (host or device memory);
 *   layer i+1 must take what layer i produces: same mb, ic = oc, ih = oh, iw = ow, else
 *   xnor_nn_error_invalid_input; every chained layer must run on the tensor-core kernels (unit
 *   stride), else xnor_nn_unimplemented.
 * The packed signs, hence every integer sum, equal those of calling the layers one after another;
 * the mean-|x| maps of layers 1.. are summed in a fixed but not strictly sequential order, so the
 * floats agree with the layer-by-layer result to rounding (about 1e-6 relative), reproducibly.
 * All work is issued on the stream of res[0]. */
xnor_nn_status_t xnor_nn_b200_forward_chain(int layers, const xnor_nn_convolution_t *const *c,
                                            void **const *res);

/* The convolution of the `forward` executor (src/default/bcast_convolution_default.cpp:60-91)
 * stopped before the alpha*K scaling: writes the signed agreement counts
 * S = 2*popcount(xnor) - op_c as int32, NCHW, mb*oc*oh*ow entries, to `sums` (host or device
 * memory). Needs binarize_weights and binarize_data to have run on `res`. This is what the
 * bit-exact parity tests compare. */
xnor_nn_status_t xnor_nn_b200_forward_sums(const xnor_nn_convolution_t *c,
                                           xnor_nn_resources_t res, int32_t *sums);

/* Copies `bytes` of internal slot `slot` (3..8) to host memory. Upstream's internal slots are
 * host arrays that tests read directly (test/gtest/test_data_bin_reference.cpp:106-121); here
 * they live on the device, so this is how a test looks at alpha, A, K and the packed words. */
xnor_nn_status_t xnor_nn_b200_read_resource(const xnor_nn_convolution_t *c,
                                            xnor_nn_resources_t res, int slot, void *host_dst,
                                            size_t bytes);

/* Work for `res` is issued on one CUDA stream, by default one the library creates. A framework
 * that owns the tensors hands in its own stream (a cudaStream_t) so that the kernels order
 * with its work; NULL goes back to the library's stream. No upstream counterpart: upstream is
 * synchronous host code. */
xnor_nn_status_t xnor_nn_b200_set_stream(xnor_nn_resources_t res, void *cuda_stream);
void *xnor_nn_b200_get_stream(xnor_nn_resources_t res);

/* Blocks until everything issued for `res` has finished. Calls that were given host pointers
 * have already waited; this is for callers that pass device pointers, and it is the call that
 * tells them of a kernel that gave up on one of its bounded waits (a call with device pointers
 * only enqueues work and returns success): xnor_nn_unimplemented then, the place in
 * xnor_nn_b200_last_error(), and the results since the previous synchronising call are invalid. */
xnor_nn_status_t xnor_nn_b200_synchronize(xnor_nn_resources_t res);

/* Text of the most recent CUDA failure seen by the calling thread ("" if none). Upstream
 * reports through the status code alone (src/status.cpp:3-15). */
const char *xnor_nn_b200_last_error(void);

/* xnor_nn_binarize_weights_float (src/binarize_weights_float.cpp:3-25: to = sign(from) *
 * mean(from), the weights the Caffe layer's backward pass convolves with,
 * external/caffe/src/caffe/layers/xnor_nn_conv_layer.cpp:97-98) for filter banks that live on the
 * device, enqueued on `cuda_stream` without waiting. The mean is summed in one fixed shape, so
 * repeated calls agree bit for bit; upstream's own sum is an OpenMP loop without a reduction
 * clause and depends on the thread schedule. `to_device` may equal `from_device`. The upstream
 * symbol itself takes this path (on the default stream, and waits) when both of its pointers are
 * device memory. */
xnor_nn_status_t xnor_nn_b200_binarize_weights_float(const xnor_nn_convolution_t *c,
                                                     const float *from_device, float *to_device,
                                                     void *cuda_stream);

/* K = box filter of mean|x| (what the calculate_k executor computes into res[k]) for callers
 * that cannot allocate device memory when they need it: code that runs while a stream is being
 * captured into a CUDA graph, servers whose arena owns all device memory, sandboxed plugins.
 * It has no counterpart in the reference and needs no xnor_nn_allocate_resources: the mean-|x|
 * scratch is a fixed array inside the library (xnor_nn_b200_noalloc_max_pixels() floats, 4 MiB,
 * held by every GPU that loads the library). `src_device` (the layer's source tensor, in the
 * descriptor's src_format) and `k_device` (mb*oh*ow floats) are device memory the caller already
 * owns; the work is enqueued on `cuda_stream` (a cudaStream_t, NULL = default stream).
 * Limits: mb*ih*iw above the maximum is refused with xnor_nn_error_invalid_input; all calls on a
 * device share the one array, so calls that overlap on the GPU race and must be serialised by the
 * caller; the first call on a device resolves the array's address and should be made before any
 * stream capture starts. Calls no cudaMalloc/cudaFree. */
xnor_nn_status_t xnor_nn_b200_calculate_k_noalloc(const xnor_nn_convolution_t *c,
                                                  const float *src_device, float *k_device,
                                                  void *cuda_stream);
long xnor_nn_b200_noalloc_max_pixels(void);
const char *xnor_nn_b200_noalloc_last_error(void);

/* One forward pass (binarize_data, calculate_k, forward) of a host minibatch spread over several
 * GPUs of this machine. Upstream serves the whole minibatch with a single Convolution::forward
 * (include/xnor_nn.hpp:45-53) whose executors spread the images over all cores, the minibatch
 * being their outermost loop (src/default/bcast_convolution_default.cpp:60-64); here device i of
 * `n_devices` takes images [mb*i/n, mb*(i+1)/n), a contiguous slice, through its own upload /
 * kernel / download pipeline, and the results land in the caller's one res[user_dst]: no peer
 * access, no collective, the gather is the downloads.
 *   res[user_src], res[user_dst]: host memory (pinned memory lets the devices' transfers overlap;
 *   pageable memory works but serialises them);
 *   res[user_weights]: host memory, needed when the device list is new (each device packs the
 *   weights for itself and keeps them); when it is non-NULL on a later call the weights are
 *   packed again, so clear the slot between passes as upstream's wrapper clears its slots;
 *   devices: CUDA ordinals, no repeats; n_devices = 0 releases the per-device replicas (so does
 *   xnor_nn_free_resources). `c`/`res` must have been initialised and allocated as usual (on any
 *   device); the call does not touch their internal slots.
 * Errors: a device ordinal that is not present, device pointers in the user slots ->
 * xnor_nn_error_invalid_input; allocation failure on a device -> xnor_nn_error_memory. */
xnor_nn_status_t xnor_nn_b200_forward_sharded(const xnor_nn_convolution_t *c,
                                              xnor_nn_resources_t res, const int *devices,
                                              int n_devices);

/* Test hook for the kernels' failure detection; not for production use. Runs the convolution of
 * the `forward` executor on res (tensor-core kernels only, res[user_dst] device memory) with the
 * kernels' wait limit shortened to `wait_ms` milliseconds (1..1000) while one thread block leaves
 * out the signal that publishes its first result tile. The warps waiting for that tile give up
 * when the limit expires, the whole kernel winds down and returns by itself, and the call reports
 * what every synchronising call reports after a give-up: xnor_nn_unimplemented, with the place
 * in xnor_nn_b200_last_error(). res[user_dst] holds garbage afterwards; the resources stay
 * usable. No upstream counterpart (upstream cannot time out). */
xnor_nn_status_t xnor_nn_b200_selftest_lost_commit(const xnor_nn_convolution_t *c,
                                                   xnor_nn_resources_t res, unsigned wait_ms);

/* Number of kernels this library has launched in this process, for benchmark accounting. */
long xnor_nn_b200_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* XNOR_NN_B200_H */
