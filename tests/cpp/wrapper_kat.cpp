// Drives the C++ wrapper the way upstream's own convolution test does
// (test/gtest/test_convolution_reference_forward.cpp): 1x2x3x3 input, two 3x3 filters, pad 1,
// all four layout combinations, result compared with the known answer within upstream's 1e-3.
// Also checks the error path (a non-success status arrives as a thrown std::runtime_error*).
// Exit code 0 = pass. Needs a CUDA device.
#include <cmath>
#include <cstdio>

#include "xnor_nn.hpp"

static const float P = 1.f, N = -1.f;

int main() {
    const float src_nchw[] = {P, P, P, N, P, N, N, N, N, N, N, N, N, N, N, P, P, P};
    const float src_nhwc[] = {P, N, P, N, P, N, N, N, P, N, N, N, N, P, N, P, N, P};
    const float w_oihw[] = {P, P, P, N, N, P, P, N, N, P, P, P, P, P, P, P, P, P,
                            N, N, N, N, N, N, N, N, N, P, P, P, N, N, P, P, N, N};
    const float w_hwio[] = {P, N, P, P, P, N, P, P, P, N, P, P, N, N, P, N, N, N,
                            P, N, P, N, P, P, P, N, P, P, N, N, P, N, N, N, P, N};
    const float want_nchw[] = {-16, -48, -16, 24, 0, 0, 0, 0, 8, 0, 0, 0, -24, -18, 0, 0, 0, -8};
    const float want_nhwc[] = {-16, 0, -48, 0, -16, 0, 24, -24, 0, -18, 0, 0, 0, 0, 0, 0, 8, -8};
    int bad = 0;
    try {
        for (int combo = 0; combo < 4; combo++) {
            const bool tf_in = combo & 2, nhwc_out = combo & 1;
            xnor_nn::Convolution conv{xnor_nn_algorithm_reference,
                                      tf_in ? xnor_nn_data_format_nhwc : xnor_nn_data_format_nchw,
                                      tf_in ? xnor_nn_weights_format_hwio : xnor_nn_weights_format_oihw,
                                      nhwc_out ? xnor_nn_data_format_nhwc : xnor_nn_data_format_nchw,
                                      1, 2, 2, 3, 3, 3, 3, 1, 1, 1, 1, tf_in ? w_hwio : w_oihw};
            float dst[18] = {0};
            conv.forward(tf_in ? src_nhwc : src_nchw, dst);
            for (int i = 0; i < 18; i++) {
                const float want = (nhwc_out ? want_nhwc : want_nchw)[i] / 9.f;
                if (std::fabs(dst[i] - want) > 1e-3f) {
                    printf("combo %d element %d: got %g want %g\n", combo, i, dst[i], want);
                    bad++;
                }
            }
        }
    } catch (std::runtime_error *e) {
        printf("unexpected failure: %s\n", e->what());
        return 2;
    }
    // unknown tensor format: upstream's executors answer `unimplemented`, the wrapper throws
    bool thrown = false;
    try {
        xnor_nn::Convolution conv{xnor_nn_algorithm_bcast, (xnor_nn_tensor_format_t)7,
                                  xnor_nn_weights_format_oihw, xnor_nn_data_format_nchw,
                                  1, 2, 2, 3, 3, 3, 3, 1, 1, 1, 1, w_oihw};
    } catch (std::runtime_error *e) {
        thrown = std::string(e->what()) == "unimplemented";
        delete e;
    }
    if (!thrown) { printf("missing exception for an unknown format\n"); bad++; }
    printf(bad ? "FAILED\n" : "ok\n");
    return bad != 0;
}
