/*
 * xnor_nn C interface, B200 build.
 *
 * Binary-compatible with the upstream xnor_nn headers (include/xnor_nn.h:12-29 and
 * include/xnor_nn_types.h:10-83): same symbol names, same enumerator values, same field order
 * in xnor_nn_convolution_t, same nine-slot resource array. A program compiled against the
 * upstream headers links against this library unchanged.
 *
 * What differs is where the work happens. The four executors run CUDA kernels on one B200.
 * The three user slots (src, weights, dst) may hold host pointers, in which case every executor
 * stages its operands through the device and returns only when the host-visible result is
 * complete, or device pointers, in which case nothing is staged. The six internal slots are
 * device allocations: host code must not dereference them. There is no CPU fallback; every call
 * fails with a status code when the CUDA device is unusable.
 */
#ifndef XNOR_NN_H
#define XNOR_NN_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (upstream include/xnor_nn_types.h:10-15) ---------------------------- */
typedef enum {
    xnor_nn_success = 0,             /* "success"        */
    xnor_nn_error_memory = 1,        /* "memory_error": a device or pinned allocation failed */
    xnor_nn_error_invalid_input = 2, /* "bad_input": a required slot or the descriptor is NULL */
    xnor_nn_unimplemented = 3        /* "unimplemented": unknown tensor format / no CUDA device */
} xnor_nn_status_t;

/* ---- algorithm request (upstream include/xnor_nn_types.h:17-22) ------------------------
 * Both requests are served by the same GPU kernels and give the same numbers, as the two
 * upstream algorithms do with each other. */
typedef enum {
    xnor_nn_algorithm_reference = 0,
    xnor_nn_algorithm_bcast = 1,
    xnor_nn_algorithm_best = 1
} xnor_nn_algorithm_t;

/* ---- resource slots (upstream include/xnor_nn_types.h:24-38) ---------------------------
 * 0..2 belong to the caller, who sets them before and may clear them after each call.
 * 3..8 are created by xnor_nn_allocate_resources and released by xnor_nn_free_resources. */
typedef enum {
    xnor_nn_resource_user_src = 0,
    xnor_nn_resource_user_weights = 1,
    xnor_nn_resource_user_dst = 2,

    xnor_nn_resource_internal = 3,       /* first internal slot, for loops */
    xnor_nn_resource_alpha = 3,          /* fp32 [OC]: mean |w| per output channel */
    xnor_nn_resource_bin_src = 4,        /* sign-packed activations (device layout) */
    xnor_nn_resource_bin_weights = 5,    /* sign-packed weights (device layout) */
    xnor_nn_resource_a = 6,              /* fp32 [MB][IH][IW]: mean |x| over channels */
    xnor_nn_resource_k = 7,              /* fp32 [MB][OH][OW]: box-filtered A / (KH*KW) */
    xnor_nn_resource_operations_count = 8, /* int32 [OH][OW]: IC * filter taps inside the image */

    xnor_nn_resource_number = 9
} xnor_nn_resource_type_t;

/* upstream include/xnor_nn_types.h:40-45 */
typedef enum {
    xnor_nn_operation_convolution_forward = 0,
    xnor_nn_operation_binarize_weights = 1,
    xnor_nn_operation_binarize_data = 2,
    xnor_nn_operation_calculate_k = 3
} xnor_nn_operation_t;

/* upstream include/xnor_nn_types.h:47-52 */
typedef enum {
    xnor_nn_data_format_nchw = 0,
    xnor_nn_data_format_nhwc = 1,
    xnor_nn_weights_format_oihw = 2,
    xnor_nn_weights_format_hwio = 3
} xnor_nn_tensor_format_t;

typedef void *xnor_nn_resources_t[xnor_nn_resource_number];

typedef struct xnor_nn_convolution_ xnor_nn_convolution_t;

/* Every stage of the path has this shape (upstream include/xnor_nn_types.h:58-59). */
typedef xnor_nn_status_t (*xnor_nn_executor_t)(const xnor_nn_convolution_t *self,
                                               xnor_nn_resources_t res);

/* The convolution descriptor. Callers allocate it themselves (stack or heap), read oh/ow and
 * resource_size[], and call the four executors through the pointers. Field order and types
 * follow upstream include/xnor_nn_types.h:61-83 exactly. */
struct xnor_nn_convolution_ {
    xnor_nn_algorithm_t algorithm;

    int mb;
    int ic, ih, iw;
    int oc, oh, ow;
    int sh, sw;
    int kh, kw;
    int ph, pw;

    xnor_nn_tensor_format_t src_format;
    xnor_nn_tensor_format_t weights_format;
    xnor_nn_tensor_format_t dst_format;

    size_t resource_size[xnor_nn_resource_number]; /* bytes, slots 3..8 */

    xnor_nn_executor_t binarize_weights; /* weights -> packed weights + alpha          */
    xnor_nn_executor_t binarize_data;    /* src -> packed activations                  */
    xnor_nn_executor_t calculate_k;      /* src -> A and K                             */
    xnor_nn_executor_t forward;          /* packed activations x packed weights -> dst */

    void *state; /* opaque plan owned by the library, freed by xnor_nn_destroy_convolution */
};

/* Replaces upstream src/status.cpp:3-15. msg needs room for 14 bytes. */
void xnor_nn_get_status_message(char *msg, xnor_nn_status_t status);

/* Replaces upstream src/memory.cpp:23-33: creates slots 3..8 on the current CUDA device.
 * On failure every slot is released again and xnor_nn_error_memory is returned. */
xnor_nn_status_t xnor_nn_allocate_resources(const xnor_nn_convolution_t *c,
                                            xnor_nn_resources_t res);

/* Replaces upstream src/memory.cpp:35-40: releases slots 3..8 and sets them to NULL. */
void xnor_nn_free_resources(xnor_nn_resources_t res);

/* Replaces upstream src/binarize_weights_float.cpp:3-25 (helper of the training backward pass,
 * host arrays): to[i] = (from[i] >= 0 ? 1 : -1) * mean(from). With two host pointers it runs on
 * the host, summing in index order; with two device pointers it runs on the GPU (default stream,
 * waited for). One pointer of each kind is not supported. */
void xnor_nn_binarize_weights_float(const xnor_nn_convolution_t *c, const float *from,
                                    float *to);

/* Replaces upstream src/common_convolution.cpp:9-63. Note the order mb, oc, ic. Always
 * succeeds, like upstream; a missing CUDA device shows up at allocate/execute time. */
xnor_nn_status_t xnor_nn_init_convolution(xnor_nn_convolution_t *c,
                                          const xnor_nn_algorithm_t algorithm,
                                          const xnor_nn_tensor_format_t src_fmt,
                                          const xnor_nn_tensor_format_t weights_fmt,
                                          const xnor_nn_tensor_format_t dst_fmt,
                                          int mb, int oc, int ic, int ih, int iw,
                                          int kh, int kw, int sh, int sw, int ph, int pw);

/* Replaces upstream src/common_convolution.cpp:65-67. */
void xnor_nn_destroy_convolution(xnor_nn_convolution_t *c);

#ifdef __cplusplus
}
#endif
#endif /* XNOR_NN_H */
