/*
 * CPU restatement of the xnor_nn binary-convolution path. TEST INFRASTRUCTURE ONLY.
 *
 * This is the checker the GPU library is compared against; it is never linked into, loaded by
 * or called from the product library. Only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark use it.
 *
 * Parity status: PINNED. The restatement is checked (tests/test_oracle.py) against the three
 * known-answer vectors of the upstream test-suite and against outputs of the unmodified
 * upstream library compiled from its own sources (oracle/Makefile, target `ref`), both live
 * when that build is present and through the committed fixtures under tests/golden/.
 *
 * Every function names the upstream file:line it follows.
 */
#ifndef XNOR_ORACLE_H
#define XNOR_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int mb, ic, ih, iw;
    int oc, oh, ow;
    int kh, kw, sh, sw, ph, pw;
    int src_nhwc;  /* 0: NCHW source, 1: NHWC source   */
    int w_hwio;    /* 0: OIHW weights, 1: HWIO weights */
    int dst_nhwc;  /* 0: NCHW result, 1: NHWC result   */
} oracle_shape_t;

/* Fills oh/ow the way upstream does, including its use of pw for the height
 * (src/common_convolution.cpp:16-17, src/utils/utils.hpp:7-13). */
void oracle_output_dims(oracle_shape_t *s);

/* Sizes of the upstream byte layouts for a given word width (2: int16 path, 4: int32 path)
 * and number of output channels per vector (src/bcast_convolution.hpp:51-70). */
int oracle_abic(int ic, int bici);
int oracle_ico(int ic, int bici);

/* Activation sign-pack in the upstream byte layout, src/bcast_binarize_data.cpp:43-73.
 * out has mb*ih*iw*oracle_abic(ic,bici) bytes. */
void oracle_binarize_data_bytes(const oracle_shape_t *s, const float *src, int bici,
                                uint8_t *out);

/* Weight sign-pack in the upstream byte layout [OCO][KH][KW][ICO][OCI][BICI] with the tail
 * bits set to one, src/bcast_binarize_weights.cpp:54-93. out has
 * ceil(oc/oci)*kh*kw*oracle_ico(ic,bici)*oci*bici bytes. */
void oracle_binarize_weights_bytes(const oracle_shape_t *s, const float *w, int bici, int oci,
                                   uint8_t *out);

/* alpha[oc] = sum over (ic,kh,kw) ascending of |w| * (1/(IC*KH*KW)),
 * src/bcast_binarize_weights.cpp:95-115. */
void oracle_alpha(const oracle_shape_t *s, const float *w, float *alpha);

/* op_c[oh][ow] = IC * (number of filter taps inside the image),
 * src/bcast_binarize_weights.cpp:126-142. */
void oracle_operations_count(const oracle_shape_t *s, int32_t *op_c);

/* a[mb][ih][iw] = sum over ic ascending of |x| * (1/IC); k[mb][oh][ow] = sum over in-bounds
 * taps (kh,kw ascending) of a * (1/KH/KW), src/bcast_calculate_k.cpp:42-85. */
void oracle_calculate_a_k(const oracle_shape_t *s, const float *src, float *a, float *k);

/* Integer sums from the upstream byte layouts, the scalar statement of the convolution:
 * P = sum over in-bounds taps and ico of popcount(~(src_word ^ w_word)); S = 2P - op_c,
 * src/default/bcast_convolution_default.cpp:60-103. sums has mb*oc*oh*ow entries indexed
 * NCHW. oc must be a multiple of oci. */
void oracle_sums_from_bytes(const oracle_shape_t *s, const uint8_t *bin_src,
                            const uint8_t *bin_w, const int32_t *op_c, int bici, int oci,
                            int32_t *sums);

/* The same integer sums straight from the floats, the way the float-domain upstream algorithm
 * states them: +1 where the signs agree, -1 where they differ, over in-bounds taps and all
 * channels (src/reference_convolution.cpp:89-108), with the sign taken from the sign bit as
 * the packed path does (src/bcast_binarize_data.cpp:61). NCHW index order. Works for any oc. */
void oracle_sums_from_floats(const oracle_shape_t *s, const float *src, const float *w,
                             int32_t *sums);

/* dst = ((float)S * alpha[oc]) * k[mb][oh][ow], stored NCHW or NHWC,
 * src/default/bcast_convolution_default.cpp:92-103. sums is NCHW-indexed. */
void oracle_scale_store(const oracle_shape_t *s, const int32_t *sums, const float *alpha,
                        const float *k, float *dst);

/* Whole forward pass: sums_from_floats + alpha + a/k + scale_store. Any of sums_out, alpha_out,
 * a_out, k_out may be NULL. Returns 0, or -1 when a scratch allocation fails. */
int oracle_convolution(const oracle_shape_t *s, const float *src, const float *w, float *dst,
                       int32_t *sums_out, float *alpha_out, float *a_out, float *k_out);

#ifdef __cplusplus
}
#endif
#endif
