// Pipe-rate probe: the measured ceilings the convolution kernels are judged against.
//
// Runs register- and shared-memory-resident loops (no global traffic) of the three candidate
// formulations of the bit contraction and prints one JSON object with binary TOPS
// (2 ops per bit pair):
//   popc        LOP3 + POPC + IADD in the 4x8 register tile of the integer-pipe kernel
//   mma_b1      mma.sync.m16n8k256 xor.popc, the legacy binary tensor path
//   tcgen05_i8  tcgen05.mma.kind::i8 M=128 N=256 K=32 on +-1 bytes, issued by one thread per SM
//               with a commit every four instructions, as the convolution's issue loop does
// Every wait is bounded; on a timeout the status field says so.
#include <cstdint>
#include <cstdio>

#include <cuda_runtime.h>

namespace {

__global__ void popc_tile(uint32_t *out, const uint32_t *in, int iters) {
    int acc[4][8];
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 8; j++) acc[i][j] = 0;
    uint32_t a[4], w[8], m[4];
    for (int i = 0; i < 4; i++) { a[i] = in[threadIdx.x + i]; m[i] = in[i + 64] | 0xffff0000u; }
    for (int j = 0; j < 8; j++) w[j] = in[threadIdx.x + 8 + j];
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[i][j] += __popc((a[i] ^ w[j]) & m[i]);
#pragma unroll
        for (int i = 0; i < 4; i++) a[i] = a[i] * 3u + 1u;
    }
    int s = 0;
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 8; j++) s += acc[i][j];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

__global__ void mma_b1(int *out, const uint32_t *in, int iters) {
    int c[8][4];
    for (int t = 0; t < 8; t++)
        for (int i = 0; i < 4; i++) c[t][i] = 0;
    uint32_t a[4], b[2];
    for (int i = 0; i < 4; i++) a[i] = in[threadIdx.x + i];
    for (int i = 0; i < 2; i++) b[i] = in[threadIdx.x + 4 + i];
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int t = 0; t < 8; t++)
            asm volatile(
                "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.xor.popc "
                "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                : "+r"(c[t][0]), "+r"(c[t][1]), "+r"(c[t][2]), "+r"(c[t][3])
                : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    int s = 0;
    for (int t = 0; t < 8; t++)
        for (int i = 0; i < 4; i++) s += c[t][i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(128, 1) tcgen05_i8(int iters, int *err) {
    extern __shared__ uint8_t raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long done, sink;
    __shared__ uint32_t tbase;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&done)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sink)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tbase)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = tbase;
    if (threadIdx.x == 0) {
        // K-major 128-byte-swizzled tiles: A 128 x 128 B at base, B 256 x 128 B behind it
        const uint32_t sa = smem_u32(base), sb = sa + 16384;
        const uint64_t hi = (uint64_t)(64u | (1u << 14) | (2u << 29)) << 32;
        const uint64_t ad = hi | (uint64_t)(((sa >> 4) & 0x3FFF) | (1u << 16));
        const uint64_t bd = hi | (uint64_t)(((sb >> 4) & 0x3FFF) | (1u << 16));
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (32u << 17) | (8u << 24);
        for (int i = 0; i < iters; i += 4) {
#pragma unroll
            for (int k = 0; k < 4; k++)
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tm), "l"(ad + 2 * k), "l"(bd + 2 * k), "r"(idesc), "r"(1u) : "memory");
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         ::"r"(smem_u32(&sink)) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     ::"r"(smem_u32(&done)) : "memory");
        const unsigned long long t0 = global_ns();
        while (!try_wait(smem_u32(&done), 0))
            if (global_ns() - t0 > 2000000000ull) { *err = 1; break; }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(512u)
                     : "memory");
    }
}

template <class F>
float best_ms(F f) {
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    f();
    cudaDeviceSynchronize();
    float best = 1e30f;
    for (int r = 0; r < 3; r++) {
        cudaEventRecord(a);
        f();
        cudaEventRecord(b);
        cudaEventSynchronize(b);
        float ms;
        cudaEventElapsedTime(&ms, a, b);
        best = ms < best ? ms : best;
    }
    return best;
}

}  // namespace

int main() {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0) != cudaSuccess) {
        printf("{\"status\": \"no CUDA device\"}\n");
        return 1;
    }
    uint32_t *buf;
    int *err;
    cudaMalloc(&buf, 1 << 24);
    cudaMemset(buf, 0x5a, 1 << 24);
    cudaMalloc(&err, 4);
    cudaMemset(err, 0, 4);
    const int blocks = sms * 8, threads = 256, iters = 2000;
    const double nthreads = (double)blocks * threads;

    float ms = best_ms([&] { popc_tile<<<blocks, threads>>>(buf, buf + 4096, iters / 4); });
    const double popc_tops = nthreads * (iters / 4) * 32 * 64 / (ms * 1e-3) / 1e12;

    ms = best_ms([&] { mma_b1<<<blocks, threads>>>((int *)buf, buf + 4096, iters / 4); });
    const double b1_tops = (double)blocks * (threads / 32) * (iters / 4) * 8 * (2.0 * 16 * 8 * 256) /
                           (ms * 1e-3) / 1e12;

    cudaFuncSetAttribute(tcgen05_i8, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const int mmas = 8192;
    ms = best_ms([&] { tcgen05_i8<<<sms, 128, 130 * 1024>>>(mmas, err); });
    const double i8_tops = (double)sms * mmas * 2.0 * 128 * 256 * 32 / (ms * 1e-3) / 1e12;

    int timed_out = 0;
    cudaMemcpy(&timed_out, err, 4, cudaMemcpyDeviceToHost);
    const cudaError_t e = cudaDeviceSynchronize();
    printf("{\"popc_binary_tops\": %.1f, \"mma_b1_binary_tops\": %.1f, \"tcgen05_i8_tops\": %.1f, "
           "\"sms\": %d, \"status\": \"%s\"}\n",
           popc_tops, b1_tops, i8_tops, sms,
           e != cudaSuccess ? cudaGetErrorString(e) : (timed_out ? "tcgen05 wait timed out" : "ok"));
    return e != cudaSuccess || timed_out;
}
