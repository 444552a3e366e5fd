/*
 * CPU restatement of the xnor_nn binary-convolution path. TEST INFRASTRUCTURE ONLY: see
 * xnor_oracle.h. Parity status: PINNED against the upstream known-answer vectors and against
 * the unmodified upstream library (tests/test_oracle.py).
 *
 * Compile with -ffp-contract=off: upstream objects are generic x86-64 code without fused
 * multiply-add, and alpha, A and K below are meant to round exactly like theirs.
 */
#include "xnor_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

static int div_up(int a, int b) { return (a + b - 1) / b; }

/* src/utils/utils.hpp:7-13 with the argument upstream passes (pw in both) */
void oracle_output_dims(oracle_shape_t *s) {
    s->oh = (s->ih + 2 * s->pw - s->kh) / s->sh + 1;
    s->ow = (s->iw + 2 * s->pw - s->kw) / s->sw + 1;
}

/* src/bcast_convolution.hpp:64-70 */
int oracle_abic(int ic, int bici) { return div_up(div_up(ic, 8), bici) * bici; }
/* src/bcast_convolution.hpp:51-54 */
int oracle_ico(int ic, int bici) { return div_up(div_up(ic, bici), 8); }

/* bit 1 <=> IEEE sign bit clear (src/bcast_binarize_data.cpp:61) */
static inline unsigned sign_clear(float f) {
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    return (~u) >> 31;
}

static inline long src_index(const oracle_shape_t *s, int mb, int c, int h, int w) {
    return s->src_nhwc ? (((long)mb * s->ih + h) * s->iw + w) * s->ic + c
                       : (((long)mb * s->ic + c) * s->ih + h) * s->iw + w;
}

static inline long w_index(const oracle_shape_t *s, int oc, int c, int kh, int kw) {
    return s->w_hwio ? (((long)kh * s->kw + kw) * s->ic + c) * s->oc + oc
                     : (((long)oc * s->ic + c) * s->kh + kh) * s->kw + kw;
}

void oracle_binarize_data_bytes(const oracle_shape_t *s, const float *src, int bici,
                                uint8_t *out) {
    const int bic = div_up(s->ic, 8), abic = oracle_abic(s->ic, bici);
#pragma omp parallel for collapse(2) schedule(static)
    for (int mb = 0; mb < s->mb; mb++)
        for (int h = 0; h < s->ih; h++)
            for (int w = 0; w < s->iw; w++) {
                uint8_t *px = out + (((long)mb * s->ih + h) * s->iw + w) * abic;
                for (int b = 0; b < abic; b++) {
                    unsigned byte = 0; /* bytes past the last channel stay zero (:69-72) */
                    if (b < bic)
                        for (int i = 0; i < 8; i++) {
                            const int c = b * 8 + i;
                            /* first channel lands in the top bit; a short tail is shifted up
                             * so that the missing channels read as zero (:62-65) */
                            byte = (byte << 1) |
                                   (c < s->ic ? sign_clear(src[src_index(s, mb, c, h, w)]) : 0u);
                        }
                    px[b] = (uint8_t)byte;
                }
            }
}

void oracle_binarize_weights_bytes(const oracle_shape_t *s, const float *w, int bici, int oci,
                                   uint8_t *out) {
    const int ico_n = oracle_ico(s->ic, bici), oco_n = div_up(s->oc, oci);
#pragma omp parallel for collapse(2) schedule(static)
    for (int oco = 0; oco < oco_n; oco++)
        for (int kh = 0; kh < s->kh; kh++)
            for (int kw = 0; kw < s->kw; kw++)
                for (int ico = 0; ico < ico_n; ico++)
                    for (int o = 0; o < oci; o++)
                        for (int b = 0; b < bici; b++) {
                            unsigned byte = 0;
                            for (int i = 0; i < 8; i++) {
                                const int c = (ico * bici + b) * 8 + i;
                                /* channels that do not exist are ones, so that the xnor with
                                 * the zero activation tail gives zero (:80-88) */
                                unsigned bit = 1u;
                                if (c < s->ic)
                                    bit = sign_clear(w[w_index(s, oco * oci + o, c, kh, kw)]);
                                byte = (byte << 1) | bit;
                            }
                            out[(((((long)oco * s->kh + kh) * s->kw + kw) * ico_n + ico) * oci +
                                 o) * bici + b] = (uint8_t)byte;
                        }
}

void oracle_alpha(const oracle_shape_t *s, const float *w, float *alpha) {
    const float chw = 1.f / (s->ic * s->kh * s->kw);
#pragma omp parallel for schedule(static)
    for (int oc = 0; oc < s->oc; oc++) {
        float acc = 0.f;
        for (int c = 0; c < s->ic; c++)
            for (int kh = 0; kh < s->kh; kh++)
                for (int kw = 0; kw < s->kw; kw++)
                    acc += fabsf(w[w_index(s, oc, c, kh, kw)]) * chw;
        alpha[oc] = acc;
    }
}

static inline int tap_inside(const oracle_shape_t *s, int oh, int ow, int kh, int kw, int *ih,
                             int *iw) {
    *ih = oh * s->sh - s->ph + kh;
    *iw = ow * s->sw - s->pw + kw;
    return *ih >= 0 && *iw >= 0 && *ih < s->ih && *iw < s->iw;
}

void oracle_operations_count(const oracle_shape_t *s, int32_t *op_c) {
    for (int oh = 0; oh < s->oh; oh++)
        for (int ow = 0; ow < s->ow; ow++) {
            int n = 0, ih, iw;
            for (int kh = 0; kh < s->kh; kh++)
                for (int kw = 0; kw < s->kw; kw++)
                    if (tap_inside(s, oh, ow, kh, kw, &ih, &iw)) n += s->ic;
            op_c[oh * s->ow + ow] = n;
        }
}

void oracle_calculate_a_k(const oracle_shape_t *s, const float *src, float *a, float *k) {
    const float inv_c = 1.f / s->ic;
    const float inv_khw = 1.f / s->kh / s->kw;
#pragma omp parallel for collapse(2) schedule(static)
    for (int mb = 0; mb < s->mb; mb++)
        for (int h = 0; h < s->ih; h++)
            for (int w = 0; w < s->iw; w++) {
                float acc = 0.f;
                for (int c = 0; c < s->ic; c++)
                    acc += fabsf(src[src_index(s, mb, c, h, w)]) * inv_c;
                a[((long)mb * s->ih + h) * s->iw + w] = acc;
            }
#pragma omp parallel for collapse(2) schedule(static)
    for (int mb = 0; mb < s->mb; mb++)
        for (int oh = 0; oh < s->oh; oh++)
            for (int ow = 0; ow < s->ow; ow++) {
                float acc = 0.f;
                int ih, iw;
                for (int kh = 0; kh < s->kh; kh++)
                    for (int kw = 0; kw < s->kw; kw++)
                        if (tap_inside(s, oh, ow, kh, kw, &ih, &iw))
                            acc += a[((long)mb * s->ih + ih) * s->iw + iw] * inv_khw;
                k[((long)mb * s->oh + oh) * s->ow + ow] = acc;
            }
}

static inline unsigned load_word(const uint8_t *p, int bici) {
    /* upstream reads the byte stream as native little-endian int16/int32 words */
    unsigned v = 0;
    for (int b = 0; b < bici; b++) v |= (unsigned)p[b] << (8 * b);
    return v;
}

void oracle_sums_from_bytes(const oracle_shape_t *s, const uint8_t *bin_src,
                            const uint8_t *bin_w, const int32_t *op_c, int bici, int oci,
                            int32_t *sums) {
    const int ico_n = oracle_ico(s->ic, bici), oco_n = s->oc / oci;
    const unsigned mask = bici == 4 ? 0xffffffffu : 0xffffu;
#pragma omp parallel for collapse(2) schedule(static)
    for (int mb = 0; mb < s->mb; mb++)
        for (int oco = 0; oco < oco_n; oco++)
            for (int oh = 0; oh < s->oh; oh++)
                for (int ow = 0; ow < s->ow; ow++)
                    for (int o = 0; o < oci; o++) {
                        int p = 0, ih, iw;
                        for (int kh = 0; kh < s->kh; kh++)
                            for (int kw = 0; kw < s->kw; kw++) {
                                if (!tap_inside(s, oh, ow, kh, kw, &ih, &iw)) continue;
                                const uint8_t *a =
                                    bin_src + (((long)mb * s->ih + ih) * s->iw + iw) * ico_n * bici;
                                const uint8_t *b =
                                    bin_w + ((((long)oco * s->kh + kh) * s->kw + kw) * ico_n * oci +
                                             o) * bici;
                                for (int ico = 0; ico < ico_n; ico++) {
                                    const unsigned x = load_word(a + (long)ico * bici, bici);
                                    const unsigned y = load_word(b + (long)ico * oci * bici, bici);
                                    p += __builtin_popcount(~(x ^ y) & mask);
                                }
                            }
                        const int oc = oco * oci + o;
                        sums[(((long)mb * s->oc + oc) * s->oh + oh) * s->ow + ow] =
                            2 * p - op_c[oh * s->ow + ow];
                    }
}

void oracle_sums_from_floats(const oracle_shape_t *s, const float *src, const float *w,
                             int32_t *sums) {
    /* One 64-bit word per 64 channels; absent channels are zero on both sides, so they xor to
     * zero and drop out: S = sum over in-bounds taps of (IC - 2*popcount(x ^ y)). */
    const int wn = div_up(s->ic, 64);
    const long npix = (long)s->mb * s->ih * s->iw;
    const long ntap = (long)s->oc * s->kh * s->kw;
    uint64_t *xa = (uint64_t *)calloc((size_t)npix * wn, sizeof(uint64_t));
    uint64_t *xw = (uint64_t *)calloc((size_t)ntap * wn, sizeof(uint64_t));
    if (!xa || !xw) { free(xa); free(xw); return; }
#pragma omp parallel for collapse(2) schedule(static)
    for (int mb = 0; mb < s->mb; mb++)
        for (int h = 0; h < s->ih; h++)
            for (int x = 0; x < s->iw; x++)
                for (int c = 0; c < s->ic; c++)
                    xa[((((long)mb * s->ih + h) * s->iw + x)) * wn + c / 64] |=
                        (uint64_t)sign_clear(src[src_index(s, mb, c, h, x)]) << (c % 64);
#pragma omp parallel for schedule(static)
    for (int oc = 0; oc < s->oc; oc++)
        for (int kh = 0; kh < s->kh; kh++)
            for (int kw = 0; kw < s->kw; kw++)
                for (int c = 0; c < s->ic; c++)
                    xw[(((long)oc * s->kh + kh) * s->kw + kw) * wn + c / 64] |=
                        (uint64_t)sign_clear(w[w_index(s, oc, c, kh, kw)]) << (c % 64);
#pragma omp parallel for collapse(2) schedule(static)
    for (int mb = 0; mb < s->mb; mb++)
        for (int oc = 0; oc < s->oc; oc++)
            for (int oh = 0; oh < s->oh; oh++)
                for (int ow = 0; ow < s->ow; ow++) {
                    int acc = 0, ih, iw;
                    for (int kh = 0; kh < s->kh; kh++)
                        for (int kw = 0; kw < s->kw; kw++) {
                            if (!tap_inside(s, oh, ow, kh, kw, &ih, &iw)) continue;
                            const uint64_t *a = xa + (((long)mb * s->ih + ih) * s->iw + iw) * wn;
                            const uint64_t *b = xw + (((long)oc * s->kh + kh) * s->kw + kw) * wn;
                            int diff = 0;
                            for (int i = 0; i < wn; i++) diff += __builtin_popcountll(a[i] ^ b[i]);
                            acc += s->ic - 2 * diff;
                        }
                    sums[(((long)mb * s->oc + oc) * s->oh + oh) * s->ow + ow] = acc;
                }
    free(xa);
    free(xw);
}

void oracle_scale_store(const oracle_shape_t *s, const int32_t *sums, const float *alpha,
                        const float *k, float *dst) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int mb = 0; mb < s->mb; mb++)
        for (int oc = 0; oc < s->oc; oc++)
            for (int oh = 0; oh < s->oh; oh++)
                for (int ow = 0; ow < s->ow; ow++) {
                    const long nchw = (((long)mb * s->oc + oc) * s->oh + oh) * s->ow + ow;
                    const long at = s->dst_nhwc
                                        ? (((long)mb * s->oh + oh) * s->ow + ow) * s->oc + oc
                                        : nchw;
                    const float v = (float)sums[nchw] * alpha[oc];
                    dst[at] = v * k[((long)mb * s->oh + oh) * s->ow + ow];
                }
}

int oracle_convolution(const oracle_shape_t *s, const float *src, const float *w, float *dst,
                       int32_t *sums_out, float *alpha_out, float *a_out, float *k_out) {
    const size_t n_out = (size_t)s->mb * s->oc * s->oh * s->ow;
    int32_t *sums = sums_out ? sums_out : (int32_t *)malloc(n_out * sizeof(int32_t));
    float *alpha = alpha_out ? alpha_out : (float *)malloc((size_t)s->oc * sizeof(float));
    float *a = a_out ? a_out : (float *)malloc((size_t)s->mb * s->ih * s->iw * sizeof(float));
    float *k = k_out ? k_out : (float *)malloc((size_t)s->mb * s->oh * s->ow * sizeof(float));
    int rc = -1;
    if (sums && alpha && a && k) {
        oracle_sums_from_floats(s, src, w, sums);
        oracle_alpha(s, w, alpha);
        oracle_calculate_a_k(s, src, a, k);
        if (dst) oracle_scale_store(s, sums, alpha, k, dst);
        rc = 0;
    }
    if (!sums_out) free(sums);
    if (!alpha_out) free(alpha);
    if (!a_out) free(a);
    if (!k_out) free(k);
    return rc;
}
