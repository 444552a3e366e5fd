// The C interface: descriptor set-up, device resources, the four executors and the extension
// entry points. Everything a caller can reach is in this file; kernels are in the neighbours.
//
// Host pointers in the user slots are staged through device buffers owned by the resource
// context and the call returns once the host-visible effect is complete; device pointers are
// used in place and the call only enqueues work on the context's stream.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <unordered_map>

#include <cuda_runtime.h>

#include "xnor_nn.h"
#include "xnor_nn_b200.h"

#include "kernels.cuh"
#include "plan.hpp"

using namespace xb200;

namespace xb200 {
std::atomic<long> g_kernel_launches{0};
}

namespace {

thread_local char t_last_error[256] = "";

bool verbose() {
    static const bool v = [] {
        const char *e = getenv("XNOR_NN_VERBOSE");
        return e && e[0] == '1';
    }();
    return v;
}

xnor_nn_status_t fail(cudaError_t e, const char *what) {
    snprintf(t_last_error, sizeof t_last_error, "%s: %s", what, cudaGetErrorString(e));
    if (verbose()) printf("xnor_nn_b200: error: %s\n", t_last_error);
    (void)cudaGetLastError();  // clear the sticky-less error so later calls start clean
    if (e == cudaErrorMemoryAllocation) return xnor_nn_error_memory;
    return xnor_nn_unimplemented;
}

#define CU(call)                                          \
    do {                                                  \
        cudaError_t e__ = (call);                         \
        if (e__ != cudaSuccess) return fail(e__, #call);  \
    } while (0)

// Per-resource device context: the stream the work runs on and the staging buffers used when
// the caller's tensors live in host memory. Found through the alpha slot's device pointer.
struct ResCtx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    void *stage[3] = {nullptr, nullptr, nullptr};  // src, weights, dst
    size_t stage_bytes[3] = {0, 0, 0};
    int32_t *sums_stage = nullptr;
    size_t sums_bytes = 0;
    int *error_word = nullptr;  // device int: set by a kernel whose bounded wait ran out
    int *error_host = nullptr;  // pinned copy of it, refreshed by every synchronising call
    // What exec_binarize_data staged from a host source, for the calculate_k that follows it
    // (upstream's wrapper always calls the two back to back on one tensor,
    // include/xnor_nn.hpp:45-53): the caller's pointer, and whether res[a] already holds the
    // mean-|x| map of exactly that upload.
    const void *staged_src_user = nullptr;
    bool staged_a_valid = false;
    struct Shard;               // per-device replicas used by xnor_nn_b200_forward_sharded
    Shard *shards = nullptr;
    int n_shards = 0;
    // host-pointer pipeline: copy engines on their own streams, events to chain the slices
    static constexpr int kMaxSlices = 8;
    static constexpr size_t kSliceBytes = 4u << 20;  // smallest upload worth a slice of its own
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_in[kMaxSlices] = {}, ev_done[kMaxSlices] = {}, ev_edge = nullptr;
    cudaEvent_t ev_chain = nullptr;  // orders this context's stream before a chained call
};

struct ResCtx::Shard {
    int device = 0;
    int first = 0, count = 0;  // its images of the whole minibatch
    xnor_nn_convolution_t c = {};
    void *res[xnor_nn_resource_number] = {};
};
void free_shards(ResCtx *x);

std::mutex g_mu;
std::unordered_map<const void *, ResCtx *> g_ctx;

ResCtx *find_ctx(xnor_nn_resources_t res) {
    if (!res || !res[xnor_nn_resource_alpha]) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_ctx.find(res[xnor_nn_resource_alpha]);
    return it == g_ctx.end() ? nullptr : it->second;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Where a caller's pointer lives: host memory (to be staged), memory of `device` (used in
// place), or memory of another GPU (refused: the kernels run on the context's device and no peer
// access is set up).
enum Where { kHost, kHere, kElsewhere };
Where where_is(const void *p, int device) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return kHost;
    }
    if (at.type == cudaMemoryTypeManaged) return kHere;
    if (at.type != cudaMemoryTypeDevice) return kHost;
    return at.device == device ? kHere : kElsewhere;
}
bool on_device(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}
xnor_nn_status_t wrong_device(const char *what) {
    snprintf(t_last_error, sizeof t_last_error,
             "%s lives on another GPU than the resources it is used with", what);
    return xnor_nn_error_invalid_input;
}

xnor_nn_status_t ensure_stage(ResCtx *x, int which, size_t bytes) {
    if (x->stage_bytes[which] >= bytes) return xnor_nn_success;
    if (x->stage[which]) CU(cudaFree(x->stage[which]));
    x->stage[which] = nullptr;
    x->stage_bytes[which] = 0;
    CU(cudaMalloc(&x->stage[which], bytes));
    x->stage_bytes[which] = bytes;
    return xnor_nn_success;
}

// Device view of a read-only user tensor: the pointer itself, or a staged copy.
xnor_nn_status_t stage_in(ResCtx *x, int which, const void *user, size_t bytes,
                          const void **dev, bool *staged) {
    const Where w = where_is(user, x->device);
    if (w == kElsewhere) return wrong_device(which == 1 ? "the weights tensor" : "the source tensor");
    if (w == kHere) {
        *dev = user;
        return xnor_nn_success;
    }
    xnor_nn_status_t st = ensure_stage(x, which, bytes);
    if (st != xnor_nn_success) return st;
    CU(cudaMemcpyAsync(x->stage[which], user, bytes, cudaMemcpyHostToDevice, x->stream));
    *dev = x->stage[which];
    *staged = true;
    return xnor_nn_success;
}

// Waits for the context's stream and turns a kernel-side give-up into a status code. The error
// word comes back through pinned memory on the same stream, so the call synchronises once.
// A give-up is reported as xnor_nn_unimplemented (upstream has no status for "the device did not
// answer"); xnor_nn_b200_last_error() names the wait that ran out.
xnor_nn_status_t sync_and_check(ResCtx *x) {
    CU(cudaMemcpyAsync(x->error_host, x->error_word, sizeof(int), cudaMemcpyDeviceToHost,
                       x->stream));
    CU(cudaStreamSynchronize(x->stream));
    const int word = *x->error_host;
    if (word != 0) {
        snprintf(t_last_error, sizeof t_last_error,
                 "a kernel gave up waiting (site %d); results of this call are invalid", word);
        CU(cudaMemsetAsync(x->error_word, 0, sizeof(int), x->stream));
        *x->error_host = 0;
        return xnor_nn_unimplemented;
    }
    return xnor_nn_success;
}

const Plan *plan_of(const xnor_nn_convolution_t *c) {
    return c ? static_cast<const Plan *>(c->state) : nullptr;
}

size_t src_bytes(const Plan &p) { return (size_t)p.mb * p.ic * p.ih * p.iw * sizeof(float); }
size_t w_bytes(const Plan &p) { return (size_t)p.oc * p.ic * p.kh * p.kw * sizeof(float); }
size_t dst_elems(const Plan &p) { return (size_t)p.mb * p.oc * p.oh * p.ow; }

void log_exec(const Plan &p, const char *what) {
    if (!verbose()) return;
    printf("xnor_nn_b200: exec: %s: kernel=%s mb=%d ic=%d ih=%d iw=%d oc=%d oh=%d ow=%d "
           "kh=%d kw=%d sh=%d sw=%d ph=%d pw=%d\n",
           what, family_name(p.family), p.mb, p.ic, p.ih, p.iw, p.oc, p.oh, p.ow, p.kh, p.kw,
           p.sh, p.sw, p.ph, p.pw);
}

// ---- the four executors ------------------------------------------------------------------------

// Replaces upstream src/bcast_binarize_weights.cpp:13-145.
xnor_nn_status_t exec_binarize_weights(const xnor_nn_convolution_t *c, xnor_nn_resources_t res) {
    if (!c || !res || !res[xnor_nn_resource_user_weights] || !res[xnor_nn_resource_bin_weights] ||
        !res[xnor_nn_resource_operations_count] || !res[xnor_nn_resource_alpha])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    if (!p->formats_ok) return xnor_nn_unimplemented;
    DeviceGuard dg(x->device);
    log_exec(*p, "binarize_weights");
    const void *w = nullptr;
    bool staged = false;
    xnor_nn_status_t st =
        stage_in(x, 1, res[xnor_nn_resource_user_weights], w_bytes(*p), &w, &staged);
    if (st != xnor_nn_success) return st;
    CU(launch_binarize_weights(*p, (const float *)w, res[xnor_nn_resource_bin_weights],
                               (float *)res[xnor_nn_resource_alpha],
                               (int32_t *)res[xnor_nn_resource_operations_count], x->stream));
    if (staged) CU(cudaStreamSynchronize(x->stream));
    return xnor_nn_success;
}

// Replaces upstream src/bcast_binarize_data.cpp:13-76.
xnor_nn_status_t exec_binarize_data(const xnor_nn_convolution_t *c, xnor_nn_resources_t res) {
    if (!c || !res || !res[xnor_nn_resource_user_src] || !res[xnor_nn_resource_bin_src])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    if (!p->formats_ok) return xnor_nn_unimplemented;
    DeviceGuard dg(x->device);
    log_exec(*p, "binarize_data");
    const void *src = nullptr;
    bool staged = false;
    x->staged_src_user = nullptr;
    x->staged_a_valid = false;
    xnor_nn_status_t st = stage_in(x, 0, res[xnor_nn_resource_user_src], src_bytes(*p), &src, &staged);
    if (st != xnor_nn_success) return st;
    // A host source has just crossed PCIe: let the packing pass also leave the mean-|x| map in
    // res[a], so that the calculate_k that follows (upstream's call order) needs neither a second
    // upload nor a second pass over the source.
    float *a = staged ? (float *)res[xnor_nn_resource_a] : nullptr;
    CU(launch_binarize_data(*p, (const float *)src, res[xnor_nn_resource_bin_src], a, x->stream));
    if (staged) {
        CU(cudaStreamSynchronize(x->stream));
        if (a) {
            x->staged_src_user = res[xnor_nn_resource_user_src];
            x->staged_a_valid = true;
        }
    }
    return xnor_nn_success;
}

// Replaces upstream src/bcast_calculate_k.cpp:13-88.
xnor_nn_status_t exec_calculate_k(const xnor_nn_convolution_t *c, xnor_nn_resources_t res) {
    if (!c || !res || !res[xnor_nn_resource_user_src] || !res[xnor_nn_resource_a] ||
        !res[xnor_nn_resource_k])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    if (!p->formats_ok) return xnor_nn_unimplemented;
    DeviceGuard dg(x->device);
    log_exec(*p, "calculate_k");
    // The mean-|x| map of this very tensor is already in res[a] when binarize_data staged it a
    // moment ago (same host pointer, no call in between): only the box filter is left. The
    // shortcut is good for one call; a source changed in place between binarize_data and
    // calculate_k would not be seen, which upstream's callers never do.
    const bool reuse = x->staged_a_valid && x->staged_src_user == res[xnor_nn_resource_user_src];
    x->staged_src_user = nullptr;
    x->staged_a_valid = false;
    bool staged = false;
    if (!reuse) {
        const void *src = nullptr;
        xnor_nn_status_t st =
            stage_in(x, 0, res[xnor_nn_resource_user_src], src_bytes(*p), &src, &staged);
        if (st != xnor_nn_success) return st;
        CU(launch_mean_abs(*p, (const float *)src, (float *)res[xnor_nn_resource_a], x->stream));
    }
    CU(launch_box_filter(*p, (const float *)res[xnor_nn_resource_a],
                         (float *)res[xnor_nn_resource_k], x->stream));
    if (staged) CU(cudaStreamSynchronize(x->stream));
    return xnor_nn_success;
}

// fuse_k: the tensor-core epilogue derives K from A itself (the caller skipped the stencil).
xnor_nn_status_t run_conv(const Plan &p, ResCtx *x, xnor_nn_resources_t res, float *dst,
                          int32_t *sums, bool fuse_k = false) {
    switch (p.family) {
        case kPopc:
            CU(launch_conv_popc(p, (const uint32_t *)res[xnor_nn_resource_bin_src],
                                (const uint32_t *)res[xnor_nn_resource_bin_weights],
                                (const float *)res[xnor_nn_resource_alpha],
                                (const float *)res[xnor_nn_resource_k],
                                (const int32_t *)res[xnor_nn_resource_operations_count], dst, sums,
                                x->stream));
            return xnor_nn_success;
        case kTcgen05:
            if (p.img) {
                CU(launch_conv_tcgen05_img(p, res[xnor_nn_resource_bin_src],
                                           res[xnor_nn_resource_bin_weights],
                                           (const float *)res[xnor_nn_resource_alpha],
                                           fuse_k ? nullptr : (const float *)res[xnor_nn_resource_k],
                                           (const float *)res[xnor_nn_resource_a],
                                           (float *)res[xnor_nn_resource_k], dst, sums,
                                           x->error_word, x->stream));
                return xnor_nn_success;
            }
            CU(launch_conv_tcgen05(p, res[xnor_nn_resource_bin_src],
                                   res[xnor_nn_resource_bin_weights],
                                   (const float *)res[xnor_nn_resource_alpha],
                                   fuse_k ? nullptr : (const float *)res[xnor_nn_resource_k],
                                   (const float *)res[xnor_nn_resource_a],
                                   (float *)res[xnor_nn_resource_k], dst, sums, x->error_word,
                                   x->stream));
            return xnor_nn_success;
        default:
            snprintf(t_last_error, sizeof t_last_error, "kernel family %s is not built in",
                     family_name(p.family));
            return xnor_nn_unimplemented;
    }
}

// Replaces upstream BcastConvolution::exec (src/default/bcast_convolution_default.cpp:107-211,
// src/x86/bcast_convolution_avx.cpp:221-352).
xnor_nn_status_t exec_forward(const xnor_nn_convolution_t *c, xnor_nn_resources_t res) {
    if (!c || !res || !res[xnor_nn_resource_bin_src] || !res[xnor_nn_resource_bin_weights] ||
        !res[xnor_nn_resource_user_dst] || !res[xnor_nn_resource_k] ||
        !res[xnor_nn_resource_alpha] || !res[xnor_nn_resource_operations_count])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    if (!p->formats_ok) return xnor_nn_unimplemented;
    DeviceGuard dg(x->device);
    log_exec(*p, "forward");
    x->staged_a_valid = false;
    void *user = res[xnor_nn_resource_user_dst];
    const Where w = where_is(user, x->device);
    if (w == kElsewhere) return wrong_device("the result tensor");
    const bool direct = w == kHere;
    float *dst = (float *)user;
    if (!direct) {
        xnor_nn_status_t st = ensure_stage(x, 2, dst_elems(*p) * sizeof(float));
        if (st != xnor_nn_success) return st;
        dst = (float *)x->stage[2];
    }
    xnor_nn_status_t st = run_conv(*p, x, res, dst, nullptr);
    if (st != xnor_nn_success) return st;
    if (!direct) {
        CU(cudaMemcpyAsync(user, dst, dst_elems(*p) * sizeof(float), cudaMemcpyDeviceToHost,
                           x->stream));
        return sync_and_check(x);
    }
    return xnor_nn_success;
}

xnor_nn_status_t init_common(xnor_nn_convolution_t *c, xnor_nn_algorithm_t algorithm,
                             xnor_nn_tensor_format_t src_fmt, xnor_nn_tensor_format_t weights_fmt,
                             xnor_nn_tensor_format_t dst_fmt, int mb, int oc, int ic, int ih,
                             int iw, int kh, int kw, int sh, int sw, int ph, int pw,
                             Family family) {
    // Output extent as upstream computes it: both from pw (src/common_convolution.cpp:16-17).
    c->algorithm = algorithm;
    c->mb = mb;
    c->ic = ic; c->ih = ih; c->iw = iw;
    c->oc = oc;
    c->oh = (ih + 2 * pw - kh) / sh + 1;
    c->ow = (iw + 2 * pw - kw) / sw + 1;
    c->sh = sh; c->sw = sw;
    c->kh = kh; c->kw = kw;
    c->ph = ph; c->pw = pw;
    c->src_format = src_fmt;
    c->weights_format = weights_fmt;
    c->dst_format = dst_fmt;
    for (int i = 0; i < xnor_nn_resource_number; i++) c->resource_size[i] = 0;

    Plan *p = new (std::nothrow) Plan;
    c->state = p;
    c->binarize_weights = exec_binarize_weights;
    c->binarize_data = exec_binarize_data;
    c->calculate_k = exec_calculate_k;
    c->forward = exec_forward;
    if (!p) return xnor_nn_success;  // executors report the missing plan as bad input
    make_plan(p, c, family);
    for (int i = xnor_nn_resource_internal; i < xnor_nn_resource_number; i++)
        c->resource_size[i] = p->bytes[i];
    if (verbose())
        printf("xnor_nn_b200: init: convolution: kernel=%s mb=%d ic=%d ih=%d iw=%d oc=%d oh=%d "
               "ow=%d kh=%d kw=%d sh=%d sw=%d ph=%d pw=%d\n",
               family_name(p->family), mb, ic, ih, iw, oc, c->oh, c->ow, kh, kw, sh, sw, ph, pw);
    return xnor_nn_success;
}

}  // namespace

// ---- upstream interface ------------------------------------------------------------------------

#pragma GCC visibility push(default)
extern "C" {

void xnor_nn_get_status_message(char *msg, xnor_nn_status_t status) {
    const char *text = "unknown";
    switch (status) {
        case xnor_nn_success: text = "success"; break;
        case xnor_nn_error_memory: text = "memory_error"; break;
        case xnor_nn_error_invalid_input: text = "bad_input"; break;
        case xnor_nn_unimplemented: text = "unimplemented"; break;
    }
    strcpy(msg, text);
}

xnor_nn_status_t xnor_nn_init_convolution(xnor_nn_convolution_t *c,
                                          const xnor_nn_algorithm_t algorithm,
                                          const xnor_nn_tensor_format_t src_fmt,
                                          const xnor_nn_tensor_format_t weights_fmt,
                                          const xnor_nn_tensor_format_t dst_fmt, int mb, int oc,
                                          int ic, int ih, int iw, int kh, int kw, int sh, int sw,
                                          int ph, int pw) {
    return init_common(c, algorithm, src_fmt, weights_fmt, dst_fmt, mb, oc, ic, ih, iw, kh, kw,
                       sh, sw, ph, pw, kAuto);
}

xnor_nn_status_t xnor_nn_b200_init_convolution(xnor_nn_convolution_t *c,
                                               const xnor_nn_algorithm_t algorithm,
                                               const xnor_nn_tensor_format_t src_fmt,
                                               const xnor_nn_tensor_format_t weights_fmt,
                                               const xnor_nn_tensor_format_t dst_fmt, int mb,
                                               int oc, int ic, int ih, int iw, int kh, int kw,
                                               int sh, int sw, int ph, int pw,
                                               xnor_nn_b200_kernel_t kernel) {
    return init_common(c, algorithm, src_fmt, weights_fmt, dst_fmt, mb, oc, ic, ih, iw, kh, kw,
                       sh, sw, ph, pw, (Family)(int)kernel);
}

xnor_nn_b200_kernel_t xnor_nn_b200_kernel_of(const xnor_nn_convolution_t *c) {
    const Plan *p = plan_of(c);
    if (!p) return xnor_nn_b200_kernel_auto;
    if (p->family == kTcgen05 && p->img) return xnor_nn_b200_kernel_tcgen05_i8_rows;
    return (xnor_nn_b200_kernel_t)(int)p->family;
}

void xnor_nn_destroy_convolution(xnor_nn_convolution_t *c) {
    if (!c) return;
    delete static_cast<Plan *>(c->state);
    c->state = nullptr;
}

void xnor_nn_free_resources(xnor_nn_resources_t res) {
    if (!res) return;
    ResCtx *x = nullptr;
    if (res[xnor_nn_resource_alpha]) {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_ctx.find(res[xnor_nn_resource_alpha]);
        if (it != g_ctx.end()) {
            x = it->second;
            g_ctx.erase(it);
        }
    }
    if (x) {
        DeviceGuard dg(x->device);
        cudaStreamSynchronize(x->stream);
        for (int i = xnor_nn_resource_internal; i < xnor_nn_resource_number; i++)
            if (res[i]) cudaFree(res[i]);
        for (int i = 0; i < 3; i++)
            if (x->stage[i]) cudaFree(x->stage[i]);
        if (x->sums_stage) cudaFree(x->sums_stage);
        if (x->error_word) cudaFree(x->error_word);
        if (x->error_host) cudaFreeHost(x->error_host);
        free_shards(x);
        if (x->ev_chain) cudaEventDestroy(x->ev_chain);
        if (x->copy_in) cudaStreamDestroy(x->copy_in);
        if (x->copy_out) cudaStreamDestroy(x->copy_out);
        for (int i = 0; i < ResCtx::kMaxSlices; i++) {
            if (x->ev_in[i]) cudaEventDestroy(x->ev_in[i]);
            if (x->ev_done[i]) cudaEventDestroy(x->ev_done[i]);
        }
        if (x->ev_edge) cudaEventDestroy(x->ev_edge);
        if (x->own_stream) cudaStreamDestroy(x->own_stream);
        (void)cudaGetLastError();
        delete x;
    }
    // Slots this library did not create (no context on record) are only cleared.
    for (int i = xnor_nn_resource_internal; i < xnor_nn_resource_number; i++) res[i] = nullptr;
}

xnor_nn_status_t xnor_nn_allocate_resources(const xnor_nn_convolution_t *c,
                                            xnor_nn_resources_t res) {
    if (!c || !res) return xnor_nn_error_invalid_input;
    for (int i = xnor_nn_resource_internal; i < xnor_nn_resource_number; i++) res[i] = nullptr;
    ResCtx *x = new (std::nothrow) ResCtx;
    if (!x) return xnor_nn_error_memory;
    cudaError_t e = cudaGetDevice(&x->device);
    if (e == cudaSuccess) e = cudaStreamCreate(&x->own_stream);
    x->stream = x->own_stream;
    for (int i = xnor_nn_resource_internal; e == cudaSuccess && i < xnor_nn_resource_number; i++) {
        const size_t bytes = c->resource_size[i] ? c->resource_size[i] : 16;
        e = cudaMalloc(&res[i], bytes);
        // Zero once: the framed layouts rely on their border rows and channel tails being 0.
        if (e == cudaSuccess) e = cudaMemsetAsync(res[i], 0, bytes, x->stream);
    }
    if (e == cudaSuccess) e = cudaMalloc(&x->error_word, sizeof(int));
    if (e == cudaSuccess) e = cudaMemsetAsync(x->error_word, 0, sizeof(int), x->stream);
    if (e == cudaSuccess) e = cudaMallocHost(&x->error_host, sizeof(int));
    if (e == cudaSuccess) *x->error_host = 0;
    if (e == cudaSuccess) e = cudaStreamSynchronize(x->stream);
    if (e != cudaSuccess) {
        if (x->error_word) cudaFree(x->error_word);
        if (x->error_host) cudaFreeHost(x->error_host);
        for (int i = xnor_nn_resource_internal; i < xnor_nn_resource_number; i++) {
            if (res[i]) cudaFree(res[i]);
            res[i] = nullptr;
        }
        if (x->own_stream) cudaStreamDestroy(x->own_stream);
        delete x;
        fail(e, "xnor_nn_allocate_resources");
        return xnor_nn_error_memory;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    g_ctx[res[xnor_nn_resource_alpha]] = x;
    return xnor_nn_success;
}

// Helper of the training backward pass, upstream src/binarize_weights_float.cpp:3-25:
// to = sign(from) * mean(from). Upstream sums with an unsynchronised OpenMP reduction, so its
// result depends on the thread schedule. Host pointers: summed here in index order, which is
// what upstream computes on one thread. Device pointers (both): the kernels of weights.cu on the
// default stream, waited for, since the function cannot report anything and upstream returns
// with `to` complete. One host and one device pointer is not supported.
void xnor_nn_binarize_weights_float(const xnor_nn_convolution_t *c, const float *from,
                                    float *to) {
    if (!c || !from || !to) return;
    const int elems = c->oc * c->ic * c->kh * c->kw;
    if (on_device(from) && on_device(to)) {
        cudaError_t e = launch_binarize_weights_float(elems, from, to, nullptr);
        if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
        if (e != cudaSuccess) (void)fail(e, "binarize_weights_float");
        return;
    }
    const float scale = 1.f / elems;
    float mean = 0.f;
    for (int i = 0; i < elems; i++) mean += from[i];
    mean *= scale;
    for (int i = 0; i < elems; i++) to[i] = (from[i] >= .0f ? 1.f : -1.f) * mean;
}

// ---- extensions --------------------------------------------------------------------------------

}  // extern "C"
#pragma GCC visibility pop

namespace {

// A contiguous run of images of a plan: the same layer with a smaller minibatch, and the byte
// offset at which its data starts in every buffer. Every kernel is independent per image
// (upstream's outermost loop is the minibatch everywhere, e.g.
// src/default/bcast_convolution_default.cpp:61), so a slice is a complete problem of its own.
struct Slice {
    Plan p;
    size_t src, bin_src, a, k, dst;
};

Slice slice_of(const Plan &p, int first, int count) {
    Slice s;
    s.p = p;
    s.p.mb = count;
    s.p.q_total = (long)count * p.hp * p.wp;
    s.p.rows = p.lead + s.p.q_total + 256 + (long)p.kh * p.wp + p.kw;
    if (count != p.mb) plan_image_rows(&s.p);  // the tiling depends on the image count
    s.src = (size_t)first * p.ic * p.ih * p.iw * sizeof(float);
    s.a = (size_t)first * p.ih * p.iw * sizeof(float);
    s.k = (size_t)first * p.oh * p.ow * sizeof(float);
    s.dst = (size_t)first * p.oc * p.oh * p.ow * sizeof(float);
    s.bin_src = p.family == kPopc      ? (size_t)first * p.ih * p.iw * p.icw * sizeof(uint32_t)
                : p.family == kTcgen05 ? (size_t)first * p.hp * p.wp * p.icp
                                       : (size_t)first * p.hp * p.wp * p.icw * sizeof(uint32_t);
    return s;
}

// binarize + A, K, convolution of one slice, device pointers, on the context's stream.
xnor_nn_status_t enqueue_forward(const Slice &sl, ResCtx *x, xnor_nn_resources_t res,
                                 const float *src, float *dst) {
    xnor_nn_resources_t sub;
    for (int i = 0; i < xnor_nn_resource_number; i++) sub[i] = res[i];
    sub[xnor_nn_resource_bin_src] = (char *)res[xnor_nn_resource_bin_src] + sl.bin_src;
    sub[xnor_nn_resource_a] = (char *)res[xnor_nn_resource_a] + sl.a;
    sub[xnor_nn_resource_k] = (char *)res[xnor_nn_resource_k] + sl.k;
    CU(launch_binarize_data(sl.p, src, sub[xnor_nn_resource_bin_src],
                            (float *)sub[xnor_nn_resource_a], x->stream));
    const bool fuse_k = sl.p.family == kTcgen05;
    if (!fuse_k)
        CU(launch_box_filter(sl.p, (const float *)sub[xnor_nn_resource_a],
                             (float *)sub[xnor_nn_resource_k], x->stream));
    return run_conv(sl.p, x, sub, dst, nullptr, fuse_k);
}

// Host source and host result: the minibatch is cut into slices whose upload, kernels and
// download overlap (PCIe is full duplex and both copy engines run beside the SMs), so the call
// costs about the longer of the two transfers instead of their sum plus the kernels. A slice
// carries at least kSliceBytes of source: below that the per-slice event hops cost more than the
// overlap gains. Everything is only enqueued; the caller synchronises.
xnor_nn_status_t enqueue_host_pipelined(const Plan &p, ResCtx *x, xnor_nn_resources_t res) {
    const char *h_src = (const char *)res[xnor_nn_resource_user_src];
    char *h_dst = (char *)res[xnor_nn_resource_user_dst];
    xnor_nn_status_t st = ensure_stage(x, 0, src_bytes(p));
    if (st == xnor_nn_success) st = ensure_stage(x, 2, dst_elems(p) * sizeof(float));
    if (st != xnor_nn_success) return st;
    if (!x->copy_in) {
        CU(cudaStreamCreateWithFlags(&x->copy_in, cudaStreamNonBlocking));
        CU(cudaStreamCreateWithFlags(&x->copy_out, cudaStreamNonBlocking));
        for (int i = 0; i < ResCtx::kMaxSlices; i++) {
            CU(cudaEventCreateWithFlags(&x->ev_in[i], cudaEventDisableTiming));
            CU(cudaEventCreateWithFlags(&x->ev_done[i], cudaEventDisableTiming));
        }
        CU(cudaEventCreateWithFlags(&x->ev_edge, cudaEventDisableTiming));
    }
    long slices = (long)(src_bytes(p) / ResCtx::kSliceBytes);
    if (slices > ResCtx::kMaxSlices) slices = ResCtx::kMaxSlices;
    if (slices > p.mb) slices = p.mb;
    if (slices < 1) slices = 1;
    // the copy streams start after whatever the caller already queued on the main stream
    CU(cudaEventRecord(x->ev_edge, x->stream));
    CU(cudaStreamWaitEvent(x->copy_in, x->ev_edge, 0));
    CU(cudaStreamWaitEvent(x->copy_out, x->ev_edge, 0));
    for (int i = 0; i < slices; i++) {
        const int first = (int)((long)p.mb * i / slices);
        const int count = (int)((long)p.mb * (i + 1) / slices) - first;
        const Slice sl = slice_of(p, first, count);
        char *d_src = (char *)x->stage[0] + sl.src;
        char *d_dst = (char *)x->stage[2] + sl.dst;
        CU(cudaMemcpyAsync(d_src, h_src + sl.src, src_bytes(sl.p), cudaMemcpyHostToDevice,
                           x->copy_in));
        CU(cudaEventRecord(x->ev_in[i], x->copy_in));
        CU(cudaStreamWaitEvent(x->stream, x->ev_in[i], 0));
        st = enqueue_forward(sl, x, res, (const float *)d_src, (float *)d_dst);
        if (st != xnor_nn_success) return st;
        CU(cudaEventRecord(x->ev_done[i], x->stream));
        CU(cudaStreamWaitEvent(x->copy_out, x->ev_done[i], 0));
        CU(cudaMemcpyAsync(h_dst + sl.dst, d_dst, dst_elems(sl.p) * sizeof(float),
                           cudaMemcpyDeviceToHost, x->copy_out));
    }
    CU(cudaEventRecord(x->ev_edge, x->copy_out));
    CU(cudaStreamWaitEvent(x->stream, x->ev_edge, 0));
    return xnor_nn_success;
}

xnor_nn_status_t forward_host_pipelined(const Plan &p, ResCtx *x, xnor_nn_resources_t res) {
    const xnor_nn_status_t st = enqueue_host_pipelined(p, x, res);
    return st == xnor_nn_success ? sync_and_check(x) : st;
}

void free_shards(ResCtx *x) {
    for (int i = 0; i < x->n_shards; i++) {
        ResCtx::Shard &sh = x->shards[i];
        if (!sh.c.state) continue;
        DeviceGuard dg(sh.device);
        xnor_nn_free_resources(sh.res);
        xnor_nn_destroy_convolution(&sh.c);
    }
    delete[] x->shards;
    x->shards = nullptr;
    x->n_shards = 0;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

xnor_nn_status_t xnor_nn_b200_forward(const xnor_nn_convolution_t *c, xnor_nn_resources_t res) {
    if (!c || !res || !res[xnor_nn_resource_user_src] || !res[xnor_nn_resource_user_dst] ||
        !res[xnor_nn_resource_bin_src] || !res[xnor_nn_resource_bin_weights] ||
        !res[xnor_nn_resource_a] || !res[xnor_nn_resource_k] || !res[xnor_nn_resource_alpha] ||
        !res[xnor_nn_resource_operations_count])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    if (!p->formats_ok) return xnor_nn_unimplemented;
    DeviceGuard dg(x->device);
    log_exec(*p, "fused forward");
    x->staged_a_valid = false;
    const Where ws = where_is(res[xnor_nn_resource_user_src], x->device);
    const Where wd = where_is(res[xnor_nn_resource_user_dst], x->device);
    if (ws == kElsewhere) return wrong_device("the source tensor");
    if (wd == kElsewhere) return wrong_device("the result tensor");
    if (ws == kHost && wd == kHost && src_bytes(*p) >= 2 * ResCtx::kSliceBytes)
        return forward_host_pipelined(*p, x, res);
    const void *src = nullptr;
    bool staged = false;
    xnor_nn_status_t st = stage_in(x, 0, res[xnor_nn_resource_user_src], src_bytes(*p), &src, &staged);
    if (st != xnor_nn_success) return st;
    void *user = res[xnor_nn_resource_user_dst];
    const bool direct = on_device(user);
    float *dst = (float *)user;
    if (!direct) {
        st = ensure_stage(x, 2, dst_elems(*p) * sizeof(float));
        if (st != xnor_nn_success) return st;
        dst = (float *)x->stage[2];
    }
    st = enqueue_forward(slice_of(*p, 0, p->mb), x, res, (const float *)src, dst);
    if (st != xnor_nn_success) return st;
    if (!direct)
        CU(cudaMemcpyAsync(user, dst, dst_elems(*p) * sizeof(float), cudaMemcpyDeviceToHost,
                           x->stream));
    if (!direct || staged) return sync_and_check(x);
    return xnor_nn_success;
}

xnor_nn_status_t xnor_nn_b200_binarize(const xnor_nn_convolution_t *c, xnor_nn_resources_t res) {
    if (!c || !res || !res[xnor_nn_resource_user_src] || !res[xnor_nn_resource_bin_src] ||
        !res[xnor_nn_resource_a])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    if (!p->formats_ok) return xnor_nn_unimplemented;
    DeviceGuard dg(x->device);
    log_exec(*p, "binarize with mean-|x| map");
    x->staged_a_valid = false;
    const void *src = nullptr;
    bool staged = false;
    xnor_nn_status_t st = stage_in(x, 0, res[xnor_nn_resource_user_src], src_bytes(*p), &src, &staged);
    if (st != xnor_nn_success) return st;
    CU(launch_binarize_data(*p, (const float *)src, res[xnor_nn_resource_bin_src],
                            (float *)res[xnor_nn_resource_a], x->stream));
    if (staged) CU(cudaStreamSynchronize(x->stream));
    return xnor_nn_success;
}

xnor_nn_status_t xnor_nn_b200_forward_chain(int layers, const xnor_nn_convolution_t *const *c,
                                            void **const *res) {
    if (layers < 1 || layers > 64 || !c || !res) return xnor_nn_error_invalid_input;
    const Plan *plan[64];
    ResCtx *ctx[64];
    for (int i = 0; i < layers; i++) {
        void **r = res[i];
        if (!c[i] || !r || !r[xnor_nn_resource_bin_src] || !r[xnor_nn_resource_bin_weights] ||
            !r[xnor_nn_resource_a] || !r[xnor_nn_resource_k] || !r[xnor_nn_resource_alpha] ||
            !r[xnor_nn_resource_operations_count])
            return xnor_nn_error_invalid_input;
        plan[i] = plan_of(c[i]);
        ctx[i] = find_ctx(r);
        if (!plan[i] || !ctx[i] || ctx[i]->device != ctx[0]->device)
            return xnor_nn_error_invalid_input;
        if (!plan[i]->formats_ok) return xnor_nn_unimplemented;
    }
    void *user_src = res[0][xnor_nn_resource_user_src];
    void *user_dst = res[layers - 1][xnor_nn_resource_user_dst];
    if (!user_src || !user_dst) return xnor_nn_error_invalid_input;
    for (int i = 0; i + 1 < layers; i++) {
        const Plan &a = *plan[i], &b = *plan[i + 1];
        if (a.mb != b.mb || a.oc != b.ic || a.oh != b.ih || a.ow != b.iw)
            return xnor_nn_error_invalid_input;
        if (a.family != kTcgen05 || b.family != kTcgen05) {
            snprintf(t_last_error, sizeof t_last_error,
                     "layers %d and %d cannot be chained: both must run on the %s kernels", i,
                     i + 1, family_name(kTcgen05));
            return xnor_nn_unimplemented;
        }
    }
    if (layers == 1) return xnor_nn_b200_forward(c[0], res[0]);

    ResCtx *x = ctx[0];
    DeviceGuard dg(x->device);
    log_exec(*plan[0], "chained forward");
    // Everything runs on the first layer's stream; work the caller queued on the other layers'
    // streams (their binarize_weights, for instance) is ordered in front of it.
    for (int i = 1; i < layers; i++) {
        if (ctx[i]->stream == x->stream) continue;
        if (!ctx[i]->ev_chain)
            CU(cudaEventCreateWithFlags(&ctx[i]->ev_chain, cudaEventDisableTiming));
        CU(cudaEventRecord(ctx[i]->ev_chain, ctx[i]->stream));
        CU(cudaStreamWaitEvent(x->stream, ctx[i]->ev_chain, 0));
    }
    const void *src = nullptr;
    bool staged = false;
    xnor_nn_status_t st = stage_in(x, 0, user_src, src_bytes(*plan[0]), &src, &staged);
    if (st != xnor_nn_success) return st;
    const Plan &last = *plan[layers - 1];
    const bool direct = on_device(user_dst);
    float *dst = (float *)user_dst;
    if (!direct) {
        st = ensure_stage(x, 2, dst_elems(last) * sizeof(float));
        if (st != xnor_nn_success) return st;
        dst = (float *)x->stage[2];
    }
    CU(launch_binarize_data(*plan[0], (const float *)src, res[0][xnor_nn_resource_bin_src],
                            (float *)res[0][xnor_nn_resource_a], x->stream));
    for (int i = 0; i < layers; i++) {
        void **r = res[i];
        ChainTarget next;
        const bool emit = i + 1 < layers;
        if (emit) {
            const Plan &n = *plan[i + 1];
            next.bin_src = res[i + 1][xnor_nn_resource_bin_src];
            next.a = (float *)res[i + 1][xnor_nn_resource_a];
            next.wp = n.wp; next.hp = n.hp; next.lead = n.lead; next.icp = n.icp;
            next.inv_ic = n.inv_ic;
        }
        CU(launch_conv_tcgen05(*plan[i], r[xnor_nn_resource_bin_src],
                               r[xnor_nn_resource_bin_weights],
                               (const float *)r[xnor_nn_resource_alpha], nullptr,
                               (const float *)r[xnor_nn_resource_a],
                               (float *)r[xnor_nn_resource_k], emit ? nullptr : dst, nullptr,
                               x->error_word, x->stream, emit ? &next : nullptr));
    }
    if (!direct)
        CU(cudaMemcpyAsync(user_dst, dst, dst_elems(last) * sizeof(float), cudaMemcpyDeviceToHost,
                           x->stream));
    if (!direct || staged) return sync_and_check(x);
    return xnor_nn_success;
}

xnor_nn_status_t xnor_nn_b200_forward_sums(const xnor_nn_convolution_t *c,
                                           xnor_nn_resources_t res, int32_t *sums) {
    if (!c || !res || !sums || !res[xnor_nn_resource_bin_src] ||
        !res[xnor_nn_resource_bin_weights] || !res[xnor_nn_resource_operations_count] ||
        !res[xnor_nn_resource_alpha] || !res[xnor_nn_resource_k])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    DeviceGuard dg(x->device);
    const size_t bytes = dst_elems(*p) * sizeof(int32_t);
    const bool direct = on_device(sums);
    int32_t *dev = sums;
    if (!direct) {
        if (x->sums_bytes < bytes) {
            if (x->sums_stage) CU(cudaFree(x->sums_stage));
            x->sums_stage = nullptr;
            x->sums_bytes = 0;
            CU(cudaMalloc(&x->sums_stage, bytes));
            x->sums_bytes = bytes;
        }
        dev = x->sums_stage;
    }
    xnor_nn_status_t st = run_conv(*p, x, res, nullptr, dev);
    if (st != xnor_nn_success) return st;
    if (!direct) {
        CU(cudaMemcpyAsync(sums, dev, bytes, cudaMemcpyDeviceToHost, x->stream));
        return sync_and_check(x);
    }
    return xnor_nn_success;
}

xnor_nn_status_t xnor_nn_b200_read_resource(const xnor_nn_convolution_t *c,
                                            xnor_nn_resources_t res, int slot, void *host_dst,
                                            size_t bytes) {
    if (!c || !res || !host_dst || slot < xnor_nn_resource_internal ||
        slot >= xnor_nn_resource_number || !res[slot] || bytes > c->resource_size[slot])
        return xnor_nn_error_invalid_input;
    ResCtx *x = find_ctx(res);
    if (!x) return xnor_nn_error_invalid_input;
    DeviceGuard dg(x->device);
    CU(cudaMemcpyAsync(host_dst, res[slot], bytes, cudaMemcpyDeviceToHost, x->stream));
    CU(cudaStreamSynchronize(x->stream));
    return xnor_nn_success;
}

xnor_nn_status_t xnor_nn_b200_set_stream(xnor_nn_resources_t res, void *cuda_stream) {
    ResCtx *x = find_ctx(res);
    if (!x) return xnor_nn_error_invalid_input;
    cudaStream_t next = cuda_stream ? (cudaStream_t)cuda_stream : x->own_stream;
    if (next == x->stream) return xnor_nn_success;  // nothing to order (and legal during capture)
    DeviceGuard dg(x->device);
    CU(cudaStreamSynchronize(x->stream));  // work already issued finishes before the switch
    x->stream = next;
    return xnor_nn_success;
}

void *xnor_nn_b200_get_stream(xnor_nn_resources_t res) {
    ResCtx *x = find_ctx(res);
    return x ? (void *)x->stream : nullptr;
}

xnor_nn_status_t xnor_nn_b200_synchronize(xnor_nn_resources_t res) {
    ResCtx *x = find_ctx(res);
    if (!x) return xnor_nn_error_invalid_input;
    DeviceGuard dg(x->device);
    return sync_and_check(x);
}

const char *xnor_nn_b200_last_error(void) { return t_last_error; }

xnor_nn_status_t xnor_nn_b200_binarize_weights_float(const xnor_nn_convolution_t *c,
                                                     const float *from_device, float *to_device,
                                                     void *cuda_stream) {
    if (!c || !from_device || !to_device) return xnor_nn_error_invalid_input;
    if (!on_device(from_device) || !on_device(to_device)) return xnor_nn_error_invalid_input;
    const long elems = (long)c->oc * c->ic * c->kh * c->kw;
    if (elems <= 0) return xnor_nn_error_invalid_input;
    CU(launch_binarize_weights_float(elems, from_device, to_device, (cudaStream_t)cuda_stream));
    return xnor_nn_success;
}

long xnor_nn_b200_kernel_launches(void) { return g_kernel_launches.load(); }

xnor_nn_status_t xnor_nn_b200_forward_sharded(const xnor_nn_convolution_t *c,
                                              xnor_nn_resources_t res, const int *devices,
                                              int n_devices) {
    if (!c || !res) return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x) return xnor_nn_error_invalid_input;
    if (n_devices == 0) {  // drop the replicas
        free_shards(x);
        return xnor_nn_success;
    }
    if (!devices || n_devices < 0 || n_devices > 64 || !res[xnor_nn_resource_user_src] ||
        !res[xnor_nn_resource_user_dst])
        return xnor_nn_error_invalid_input;
    if (!p->formats_ok) return xnor_nn_unimplemented;
    int present = 0;
    CU(cudaGetDeviceCount(&present));
    for (int i = 0; i < n_devices; i++) {
        if (devices[i] < 0 || devices[i] >= present) {
            snprintf(t_last_error, sizeof t_last_error,
                     "device %d was asked for, %d are present", devices[i], present);
            return xnor_nn_error_invalid_input;
        }
        for (int j = 0; j < i; j++)
            if (devices[j] == devices[i]) return xnor_nn_error_invalid_input;
    }
    if (on_device(res[xnor_nn_resource_user_src]) || on_device(res[xnor_nn_resource_user_dst])) {
        snprintf(t_last_error, sizeof t_last_error,
                 "the sharded call takes the minibatch from, and gathers it into, host memory");
        return xnor_nn_error_invalid_input;
    }
    // (Re)build the per-device replicas: on first use, when the device list changes, and when
    // the caller has put a weights tensor into res[user_weights] again.
    bool rebuild = x->n_shards != n_devices || res[xnor_nn_resource_user_weights] != nullptr;
    for (int i = 0; !rebuild && i < n_devices; i++) rebuild = x->shards[i].device != devices[i];
    if (rebuild) {
        if (!res[xnor_nn_resource_user_weights]) {
            snprintf(t_last_error, sizeof t_last_error,
                     "res[user_weights] must hold the weights when the device list is new");
            return xnor_nn_error_invalid_input;
        }
        free_shards(x);
        x->shards = new (std::nothrow) ResCtx::Shard[n_devices];
        if (!x->shards) return xnor_nn_error_memory;
        x->n_shards = n_devices;
        for (int i = 0; i < n_devices; i++) {
            ResCtx::Shard &sh = x->shards[i];
            sh.device = devices[i];
            // contiguous image slices in minibatch order, as upstream's outermost loop walks
            // them (src/default/bcast_convolution_default.cpp:60-64)
            sh.first = (int)((long)p->mb * i / n_devices);
            sh.count = (int)((long)p->mb * (i + 1) / n_devices) - sh.first;
            if (sh.count == 0) continue;
            DeviceGuard dg(sh.device);
            xnor_nn_status_t st = init_common(
                &sh.c, c->algorithm, c->src_format, c->weights_format, c->dst_format, sh.count,
                c->oc, c->ic, c->ih, c->iw, c->kh, c->kw, c->sh, c->sw, c->ph, c->pw,
                p->family == kTcgen05 && p->img ? kTcgen05Rows : p->family);
            if (st == xnor_nn_success) st = xnor_nn_allocate_resources(&sh.c, sh.res);
            if (st == xnor_nn_success) {
                sh.res[xnor_nn_resource_user_weights] = res[xnor_nn_resource_user_weights];
                st = exec_binarize_weights(&sh.c, sh.res);
                sh.res[xnor_nn_resource_user_weights] = nullptr;
            }
            if (st != xnor_nn_success) {
                free_shards(x);
                return st;
            }
        }
    }
    // Enqueue every device's slice (upload, kernels, download on that device's streams), then
    // wait for all of them: no peer access, no collective, the gather is the downloads landing
    // in the caller's one result tensor.
    const size_t src_img = (size_t)p->ic * p->ih * p->iw * sizeof(float);
    const size_t dst_img = (size_t)p->oc * p->oh * p->ow * sizeof(float);
    xnor_nn_status_t status = xnor_nn_success;
    for (int i = 0; i < n_devices && status == xnor_nn_success; i++) {
        ResCtx::Shard &sh = x->shards[i];
        if (sh.count == 0) continue;
        DeviceGuard dg(sh.device);
        sh.res[xnor_nn_resource_user_src] =
            (char *)res[xnor_nn_resource_user_src] + (size_t)sh.first * src_img;
        sh.res[xnor_nn_resource_user_dst] =
            (char *)res[xnor_nn_resource_user_dst] + (size_t)sh.first * dst_img;
        status = enqueue_host_pipelined(*plan_of(&sh.c), find_ctx(sh.res), sh.res);
    }
    for (int i = 0; i < n_devices; i++) {
        ResCtx::Shard &sh = x->shards[i];
        if (sh.count == 0) continue;
        DeviceGuard dg(sh.device);
        const xnor_nn_status_t st = sync_and_check(find_ctx(sh.res));
        if (status == xnor_nn_success) status = st;
        sh.res[xnor_nn_resource_user_src] = nullptr;
        sh.res[xnor_nn_resource_user_dst] = nullptr;
    }
    return status;
}

xnor_nn_status_t xnor_nn_b200_selftest_lost_commit(const xnor_nn_convolution_t *c,
                                                   xnor_nn_resources_t res, unsigned wait_ms) {
    if (!c || !res || !res[xnor_nn_resource_user_dst] || !res[xnor_nn_resource_bin_src] ||
        !res[xnor_nn_resource_bin_weights] || !res[xnor_nn_resource_k] ||
        !res[xnor_nn_resource_alpha])
        return xnor_nn_error_invalid_input;
    const Plan *p = plan_of(c);
    ResCtx *x = find_ctx(res);
    if (!p || !x || p->family != kTcgen05 || wait_ms == 0 || wait_ms > 1000 ||
        where_is(res[xnor_nn_resource_user_dst], x->device) != kHere)
        return xnor_nn_error_invalid_input;
    DeviceGuard dg(x->device);
    ConvSelfTest t;
    t.wait_ns = (unsigned long long)wait_ms * 1000000ull;
    t.drop_commit = 1;
    float *dst = (float *)res[xnor_nn_resource_user_dst];
    if (p->img)
        CU(launch_conv_tcgen05_img(*p, res[xnor_nn_resource_bin_src],
                                   res[xnor_nn_resource_bin_weights],
                                   (const float *)res[xnor_nn_resource_alpha],
                                   (const float *)res[xnor_nn_resource_k], nullptr, nullptr, dst,
                                   nullptr, x->error_word, x->stream, &t));
    else
        CU(launch_conv_tcgen05(*p, res[xnor_nn_resource_bin_src],
                               res[xnor_nn_resource_bin_weights],
                               (const float *)res[xnor_nn_resource_alpha],
                               (const float *)res[xnor_nn_resource_k], nullptr, nullptr, dst,
                               nullptr, x->error_word, x->stream, nullptr, &t));
    return sync_and_check(x);
}

}  // extern "C"
#pragma GCC visibility pop
