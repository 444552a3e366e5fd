// C++ wrapper over the C interface, B200 build.
//
// Same class, constructor arguments and methods as upstream's include/xnor_nn.hpp:11-68, so code
// written against upstream compiles unchanged:
//   Convolution(...)   = xnor_nn_init_convolution + xnor_nn_allocate_resources + binarize_weights
//   forward(src, dst)  = binarize_data + calculate_k + forward on one minibatch
//   change_weights(w)  = binarize_weights again
// src/dst/weights may be host or device pointers. forward() goes through the one-upload entry
// point xnor_nn_b200_forward instead of three executor calls; the results are the same bytes.
//
// Error behaviour is upstream's (include/xnor_nn.hpp:62-67): a non-success status throws a
// heap-allocated std::runtime_error *by pointer*, with the status text as message.
#ifndef XNOR_NN_HPP
#define XNOR_NN_HPP

#include <stdexcept>
#include <string>

#include "xnor_nn.h"
#include "xnor_nn_b200.h"

namespace xnor_nn {

class Convolution {
public:
    Convolution(const xnor_nn_algorithm_t algorithm, const xnor_nn_tensor_format_t src_fmt,
                const xnor_nn_tensor_format_t weights_fmt, const xnor_nn_tensor_format_t dst_fmt,
                int MB, int OC, int IC, int IH, int IW, int KH, int KW, int SH, int SW, int PH,
                int PW, const void *weights)
        : res_{0} {
        throw_unless_ok(xnor_nn_init_convolution(&desc_, algorithm, src_fmt, weights_fmt, dst_fmt,
                                                 MB, OC, IC, IH, IW, KH, KW, SH, SW, PH, PW));
        const xnor_nn_status_t st = xnor_nn_allocate_resources(&desc_, res_);
        if (st != xnor_nn_success) {
            xnor_nn_destroy_convolution(&desc_);
            throw_unless_ok(st);
        }
        try {
            change_weights(weights);
        } catch (...) {
            release();
            throw;
        }
    }

    Convolution(const Convolution &) = delete;
    Convolution &operator=(const Convolution &) = delete;

    ~Convolution() { release(); }

    void change_weights(const void *weights) {
        res_[xnor_nn_resource_user_weights] = const_cast<void *>(weights);
        throw_unless_ok(desc_.binarize_weights(&desc_, res_));
        res_[xnor_nn_resource_user_weights] = nullptr;
    }

    void binarizeWeightsFloat(const void *from, void *to) {
        xnor_nn_binarize_weights_float(&desc_, static_cast<const float *>(from),
                                       static_cast<float *>(to));
    }

    void forward(const void *src, void *dst) {
        res_[xnor_nn_resource_user_src] = const_cast<void *>(src);
        res_[xnor_nn_resource_user_dst] = dst;
        const xnor_nn_status_t st = xnor_nn_b200_forward(&desc_, res_);
        res_[xnor_nn_resource_user_src] = nullptr;
        res_[xnor_nn_resource_user_dst] = nullptr;
        throw_unless_ok(st);
    }

    // Output extent the library derived (upstream callers read it from the descriptor too).
    int oh() const { return desc_.oh; }
    int ow() const { return desc_.ow; }

private:
    xnor_nn_convolution_t desc_;
    xnor_nn_resources_t res_;

    void release() {
        xnor_nn_free_resources(res_);
        xnor_nn_destroy_convolution(&desc_);
    }

    static void throw_unless_ok(xnor_nn_status_t st) {
        if (st == xnor_nn_success) return;
        char text[16] = {0};
        xnor_nn_get_status_message(text, st);
        throw new std::runtime_error{std::string(text)};
    }
};

}  // namespace xnor_nn
#endif  // XNOR_NN_HPP
