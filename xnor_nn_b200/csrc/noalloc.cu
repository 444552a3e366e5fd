// xnor_nn_b200_calculate_k_noalloc: the K map for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need K: code running
// while a stream is being captured into a CUDA graph (allocation is illegal there), inference
// servers that hand every byte of device memory to their own arena at start-up and treat a later
// driver allocation as a fault, and plugin sandboxes whose allocator hooks reject foreign
// allocations. The regular path needs xnor_nn_allocate_resources for its scratch (the mean-|x|
// map A that the box filter reads). This entry point instead keeps A in a fixed array that is
// part of the library image, so every GPU that loads the library holds kNoAllocMaxPixels floats
// (4 MiB) until the process exits.
//
// Consequences the caller has to know about:
//   * one array per device, shared by every call: calls that overlap on the GPU (different
//     streams, different threads) race on it and must be serialised by the caller;
//   * the array keeps the previous call's values; nothing relies on it starting at zero, because
//     every pixel the box filter reads is rewritten by the same call first;
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress). Make
//     that first call before any stream capture begins.
#include <atomic>
#include <cstdio>

#include <cuda_runtime.h>

#include "xnor_nn.h"
#include "xnor_nn_b200.h"

#include "kernels.cuh"
#include "plan.hpp"

namespace {

constexpr long kNoAllocMaxPixels = 1L << 20;  // mb*ih*iw the scratch can hold (4 MiB of floats)
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime, not a device address: the pointer the
// kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_a[kNoAllocMaxPixels];

std::atomic<float *> g_scratch_of_device[kMaxDevices];  // filled on the first call per device

thread_local char t_noalloc_error[200] = "";

// Device memory of GPU `dev` (or managed memory): what the kernels, which run on the current
// device without peer access, can read and write.
bool device_pointer(const void *p, int dev) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeManaged || (at.type == cudaMemoryTypeDevice && at.device == dev);
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

xnor_nn_status_t xnor_nn_b200_calculate_k_noalloc(const xnor_nn_convolution_t *c,
                                                  const float *src_device, float *k_device,
                                                  void *cuda_stream) {
    using namespace xb200;
    t_noalloc_error[0] = 0;
    if (!c || !c->state || !src_device || !k_device) return xnor_nn_error_invalid_input;
    const Plan &p = *static_cast<const Plan *>(c->state);
    if (!p.formats_ok) return xnor_nn_unimplemented;
    const long pixels = (long)p.mb * p.ih * p.iw;
    if (pixels > kNoAllocMaxPixels) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error,
                 "calculate_k_noalloc: mb*ih*iw = %ld exceeds the built-in scratch of %ld pixels",
                 pixels, kNoAllocMaxPixels);
        return xnor_nn_error_invalid_input;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return xnor_nn_unimplemented;
    }
    if (!device_pointer(src_device, dev) || !device_pointer(k_device, dev)) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error,
                 "calculate_k_noalloc: src and k must be memory of the current device "
                 "(nothing is staged, no peer access is set up)");
        return xnor_nn_error_invalid_input;
    }
    if (!g_scratch_of_device[dev].load(std::memory_order_acquire)) {
        // once per device, with that device current
        float *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_a);
        if (e != cudaSuccess || !ptr) {
            snprintf(t_noalloc_error, sizeof t_noalloc_error, "cudaGetSymbolAddress: %s",
                     cudaGetErrorString(e));
            (void)cudaGetLastError();
            return xnor_nn_unimplemented;
        }
        g_scratch_of_device[dev].store(ptr, std::memory_order_release);
    }
    float *a = g_scratch_of_device[dev].load(std::memory_order_acquire);
    cudaStream_t s = (cudaStream_t)cuda_stream;
    cudaError_t e = launch_mean_abs(p, src_device, a, s);
    if (e == cudaSuccess) e = launch_box_filter(p, a, k_device, s);
    if (e != cudaSuccess) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error, "calculate_k_noalloc: %s",
                 cudaGetErrorString(e));
        (void)cudaGetLastError();
        return xnor_nn_unimplemented;
    }
    return xnor_nn_success;
}

long xnor_nn_b200_noalloc_max_pixels(void) { return kNoAllocMaxPixels; }

const char *xnor_nn_b200_noalloc_last_error(void) { return t_noalloc_error; }

}  // extern "C"
#pragma GCC visibility pop
