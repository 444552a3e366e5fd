// Cost of the instructions the tensor-core convolution kernels are built from, measured on the
// device at hand. Stand-alone program (built next to pipe_probe); prints one JSON line.
//
//   mma_group_cycles   cycles one thread needs for [4 x tcgen05.mma kind::i8, 1 x tcgen05.commit]
//                      at several N: the tensor pipe needs N/2 cycles per instruction, the issue
//                      side has a floor of its own (the commit dominates it)
//   mma_group_cycles_two_issuers
//                      the same number of groups dealt to two threads of different warps that
//                      accumulate into the same tensor memory: cycles per group for the pair
//   tma_stage_cycles   cycles per pipeline stage of a free-running TMA producer (one 128x128-byte
//                      tile + one 4-D box of 169 rows, ring of four buffers), one SM and all SMs
//   store_cycles       cycles per global store instruction of one warp, by access pattern
//   bulk_store         a 21.6 KB shared->global bulk store alone and beside the TMA producer
//   umma_row_offset    whether a UMMA descriptor that starts r rows (r x 128 B, r = 0..7) into a
//                      128-byte-swizzled tile reads rows r .. r+127 of it (what lets one position
//                      tile with a halo serve all taps of a filter row): wrong results per r
//
// Every wait in here is bounded (2 s), no kernel waits on another.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../tc_ptx.cuh"

using namespace xb200::tc;

namespace {

constexpr unsigned long long kLimitNs = 2000000000ull;

__device__ bool wait_bounded(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_ns();
    while (!mbar_try_wait(bar, parity))
        if (global_ns() - t0 > kLimitNs) return false;
    return true;
}

// ---- [4 MMA + commit] ----------------------------------------------------------------------------
__global__ void __launch_bounds__(96, 1)
mma_groups(int n, int groups, int issuers, long long *out, int *err) {
    extern __shared__ uint8_t raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long done_s[2], sink_s[2];
    __shared__ uint32_t tm_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; i++) {
            mbar_init(smem_u32(&done_s[i]), 1);
            mbar_init(smem_u32(&sink_s[i]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tm_s), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tm = tm_s;
    if (warp >= 1 && warp - 1 < issuers && lane == 0) {
        unsigned long long &done = done_s[warp - 1], &sink = sink_s[warp - 1];
        groups /= issuers;
        const uint32_t sa = smem_u32(base) + (uint32_t)(warp - 1) * 49152u, sb = sa + 16384;
        const uint64_t hi = (uint64_t)(64u | (1u << 14) | (2u << 29)) << 32;
        const uint64_t ad = hi | (uint64_t)(((sa >> 4) & 0x3FFF) | (1u << 16));
        const uint64_t bd = hi | (uint64_t)(((sb >> 4) & 0x3FFF) | (1u << 16));
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (8u << 24);
        const long long t0 = clock64();
        for (int i = 0; i < groups; i++) {
#pragma unroll
            for (int k = 0; k < 4; k++) mma_i8(tm, ad + 2 * k, bd + 2 * k, idesc, 1u);
            commit(smem_u32(&sink));
        }
        commit(smem_u32(&done));
        if (!wait_bounded(smem_u32(&done), 0)) *err = 1;
        if (blockIdx.x == 0) out[warp - 1] = clock64() - t0;
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_free(tm, 512);
    }
}

// ---- TMA producer, optionally beside a warp that issues bulk stores --------------------------------
struct FeedArgs {
    int load_iters, store_iters;
    uint32_t store_bytes;
    int loads, stores;
};
__global__ void __launch_bounds__(96, 1)
feed(const __grid_constant__ CUtensorMap tile, const __grid_constant__ CUtensorMap box, FeedArgs a,
     uint8_t *gout, long long *out, int *err) {
    extern __shared__ uint8_t raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long bar[4];
    constexpr uint32_t kStage = 16384 + 22528;
    uint8_t *sbuf = base + 4 * kStage;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; i++) mbar_init(smem_u32(&bar[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0 && lane == 0 && a.loads) {
        uint32_t phase = 0;
        int s = 0;
        bool ok = true;
        const long long t0 = clock64();
        int issued = 0;
        for (; ok && issued < a.load_iters; issued++) {
            if (issued >= 4) ok = wait_bounded(smem_u32(&bar[s]), phase ^ 1);
            if (!ok) break;
            mbar_expect_tx(smem_u32(&bar[s]), 16384 + 21632);
            const uint32_t dst = smem_u32(base) + s * kStage;
            tma_load_2d(dst, &tile, 0, 16 + (issued % 7) * 8, smem_u32(&bar[s]));
            tma_load_4d(dst + 16384, &box, 0, -1, -1, 1 + (issued % 7) + (int)blockIdx.x, smem_u32(&bar[s]));
            if (++s == 4) { s = 0; phase ^= 1; }
        }
        for (int j = 0; j < 4 && j < issued; j++) {  // what is still in flight
            const int gi = issued - 1 - j;
            if (!wait_bounded(smem_u32(&bar[gi % 4]), (uint32_t)((gi / 4) & 1))) ok = false;
        }
        if (!ok) *err = 2;
        if (blockIdx.x == 0) out[0] = clock64() - t0;
    }
    if (warp == 1 && a.stores) {
        const long long t0 = clock64();
        for (int i = 0; i < a.store_iters; i++) {
            uint8_t *dst = gout + ((size_t)blockIdx.x * 64 + (i % 64)) * 32768;
            if (lane == 0) {
                bulk_store(dst, smem_u32(sbuf), a.store_bytes);
                bulk_commit();
                bulk_wait_read();
            }
            __syncwarp();
        }
        if (lane == 0) bulk_wait_all();
        if (blockIdx.x == 0 && lane == 0) out[1] = clock64() - t0;
    }
}

// ---- global stores ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(512, 1)
stores(uint8_t *out, int pattern, int warps, int iters, long long *res) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= warps) return;
    uint8_t *base = out + ((size_t)blockIdx.x * 16 + warp) * (512u << 10);
    const uint4 v = make_uint4(lane, warp, 3, 4);
    const long long t0 = clock64();
    for (int i = 0; i < iters; i++) {
        uint8_t *p;
        switch (pattern) {
            case 0: p = base + (size_t)i * 128 + lane * 4; *reinterpret_cast<uint32_t *>(p) = v.x; break;
            case 1: p = base + (size_t)i * 512 + lane * 16; *reinterpret_cast<uint4 *>(p) = v; break;
            case 2: p = base + (size_t)i * 1024 + lane * 32;
                    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%1,%2,%3,%4};"
                                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                    break;
            default: p = base + (size_t)lane * 2704 + i * 16; *reinterpret_cast<uint4 *>(p) = v; break;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) res[0] = clock64() - t0;
}

// ---- a descriptor that starts r rows into a swizzled tile ---------------------------------------
// A[m][k] known bytes (136 rows), B[n][k] = 1 at k == n and 2 at k == n + 32 (32 rows), K = 64:
// D[m][n] = A[m + r][n] + 2 A[m + r][n + 32] if the descriptor reads rows r .. r + 127.
__global__ void __launch_bounds__(128, 1)
row_offset(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
           int r, int32_t *out, int *err) {
    extern __shared__ uint8_t raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long full, done;
    __shared__ uint32_t tm_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&full), 1);
        mbar_init(smem_u32(&done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tm_s), 32);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tm = tm_s;
    const uint32_t sa = smem_u32(base), sb = sa + 136 * 128;
    if (threadIdx.x == 0) {
        mbar_expect_tx(smem_u32(&full), 136 * 128 + 32 * 128);
        tma_load_2d(sa, &map_a, 0, 0, smem_u32(&full));
        tma_load_2d(sb, &map_b, 0, 0, smem_u32(&full));
        if (!wait_bounded(smem_u32(&full), 0)) *err = 3;
        fence_after();
        const uint64_t hi = (uint64_t)(64u | (1u << 14) | (2u << 29)) << 32;
        const uint64_t ad = hi | (uint64_t)((((sa + r * 128) >> 4) & 0x3FFF) | (1u << 16));
        const uint64_t bd = hi | (uint64_t)(((sb >> 4) & 0x3FFF) | (1u << 16));
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(32 >> 3) << 17) | (8u << 24);
        mma_i8(tm, ad, bd, idesc, 0u);
        mma_i8(tm, ad + 2, bd + 2, idesc, 1u);
        commit(smem_u32(&done));
        if (!wait_bounded(smem_u32(&done), 0)) *err = 4;
    }
    __syncthreads();
    fence_after();
    uint32_t v[32];
    ld32(tm + ((uint32_t)(warp * 32) << 16), v);
    wait_ld();
    for (int j = 0; j < 32; j++) out[(warp * 32 + lane) * 32 + j] = (int)v[j];
    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_free(tm, 32);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

int main() {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0) != cudaSuccess) {
        printf("{\"status\": \"no CUDA device\"}\n");
        return 1;
    }
    void *fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q);
    EncodeTiledFn enc = (EncodeTiledFn)fp;
    long long *out;
    int *err;
    cudaMalloc(&out, 64);
    cudaMalloc(&err, 4);
    cudaMemset(err, 0, 4);
    long long h[2];
    printf("{");

    // [4 MMA + commit]
    cudaFuncSetAttribute(mma_groups, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    printf("\"mma_group_cycles\": {");
    const int ns[] = {64, 128, 176, 208, 256};
    for (int issuers = 1; issuers <= 2; issuers++) {
        if (issuers == 2) printf("\"mma_group_cycles_two_issuers\": {");
        for (int i = 0; i < 5; i++) {
            for (int rep = 0; rep < 2; rep++) {
                cudaMemset(out, 0, 16);
                mma_groups<<<sms, 96, 130 * 1024>>>(ns[i], 2048, issuers, out, err);
                cudaDeviceSynchronize();
            }
            cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost);
            const long long t = h[0] > h[1] ? h[0] : h[1];
            printf("%s\"N=%d\": %.0f", i ? ", " : "", ns[i], t / 2048.0);
        }
        printf("}, ");
    }

    // TMA producer and bulk stores
    const int icp = 384, wp = 14, hp = 14, mb = 512;
    uint8_t *d, *gout;
    cudaMalloc(&d, (size_t)icp * wp * hp * mb + (1 << 20));
    cudaMemset(d, 1, (size_t)icp * wp * hp * mb + (1 << 20));
    cudaMalloc(&gout, (size_t)sms * 64 * 32768);
    cudaFuncSetAttribute(feed, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap tile, box;
    const cuuint64_t d2[2] = {icp, (cuuint64_t)wp * hp * mb}, s2[1] = {icp};
    const cuuint32_t b2[2] = {128, 128};
    const cuuint64_t d4[4] = {icp, wp, hp, mb}, s4[3] = {icp, icp * wp, icp * wp * hp};
    const cuuint32_t b4[4] = {128, 13, 13, 1};
    if (!enc || enc(&tile, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, d, d2, s2, b2, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
        enc(&box, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, d, d4, s4, b4, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
        printf("\"status\": \"tensor map encoding failed\"}\n");
        return 1;
    }
    const size_t feed_smem = 4 * (16384 + 22528) + 32768 + 2048;
    auto run_feed = [&](int grid, int loads, int stores_on) {
        FeedArgs a;
        a.load_iters = 432; a.store_iters = 64; a.store_bytes = 21632; a.loads = loads; a.stores = stores_on;
        cudaMemset(out, 0, 16);
        for (int rep = 0; rep < 2; rep++) {
            feed<<<grid, 96, feed_smem>>>(tile, box, a, gout, out, err);
            cudaDeviceSynchronize();
        }
        cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost);
    };
    run_feed(1, 1, 0);
    printf("\"tma_stage_cycles\": {\"bytes_per_stage\": 38016, \"one_sm\": %.0f, ", h[0] / 432.0);
    run_feed(sms, 1, 0);
    printf("\"all_sms\": %.0f}, ", h[0] / 432.0);
    run_feed(sms, 0, 1);
    printf("\"bulk_store\": {\"bytes\": 21632, \"alone_cycles\": %.0f, ", h[1] / 64.0);
    run_feed(sms, 1, 1);
    printf("\"beside_tma_loads_cycles\": %.0f, \"tma_stage_cycles_beside_stores\": %.0f}, ",
           h[1] / 64.0, h[0] / 432.0);

    // global stores
    uint8_t *sout;
    cudaMalloc(&sout, (size_t)sms * 16 * (512u << 10));
    const char *names[] = {"scalar_128B_contiguous", "v4_512B_contiguous", "v8_1KB_contiguous",
                           "v4_lanes_2704B_apart"};
    printf("\"store_cycles\": {");
    bool first = true;
    for (int warps : {1, 4, 16})
        for (int pattern = 0; pattern < 4; pattern++) {
            for (int rep = 0; rep < 2; rep++) {
                stores<<<sms, 512>>>(sout, pattern, warps, 256, out);
                cudaDeviceSynchronize();
            }
            cudaMemcpy(h, out, 8, cudaMemcpyDeviceToHost);
            printf("%s\"%s/%d_warps\": %.0f", first ? "" : ", ", names[pattern], warps, h[0] / 256.0);
            first = false;
        }
    printf("}, ");

    // descriptor row offsets
    {
        static int8_t ha[160 * 128], hb[32 * 128];
        for (int m = 0; m < 160; m++)
            for (int k = 0; k < 128; k++) ha[m * 128 + k] = (int8_t)((m * 7 + k * 3) % 11 - 5);
        memset(hb, 0, sizeof hb);
        for (int n = 0; n < 32; n++) { hb[n * 128 + n] = 1; hb[n * 128 + n + 32] = 2; }
        int8_t *da, *db;
        int32_t *dout;
        cudaMalloc(&da, sizeof ha);
        cudaMalloc(&db, sizeof hb);
        cudaMalloc(&dout, 128 * 32 * 4);
        cudaMemcpy(da, ha, sizeof ha, cudaMemcpyHostToDevice);
        cudaMemcpy(db, hb, sizeof hb, cudaMemcpyHostToDevice);
        CUtensorMap ma, mb2;
        const cuuint64_t da2[2] = {128, 160}, db2[2] = {128, 32}, st[1] = {128};
        const cuuint32_t ba[2] = {128, 136}, bb[2] = {128, 32};
        printf("\"umma_row_offset_wrong_results\": {");
        if (enc(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, da, da2, st, ba, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS &&
            enc(&mb2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, db, db2, st, bb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
            cudaFuncSetAttribute(row_offset, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
            static int32_t ho[128 * 32];
            for (int r = 0; r < 8; r++) {
                row_offset<<<1, 128, 64 * 1024>>>(ma, mb2, r, dout, err);
                cudaDeviceSynchronize();
                cudaMemcpy(ho, dout, sizeof ho, cudaMemcpyDeviceToHost);
                int bad = 0;
                for (int m = 0; m < 128; m++)
                    for (int n = 0; n < 32; n++)
                        bad += ho[m * 32 + n] != ha[(m + r) * 128 + n] + 2 * ha[(m + r) * 128 + n + 32];
                printf("%s\"r=%d\": %d", r ? ", " : "", r, bad);
            }
        }
        printf("}, ");
    }

    int flagged = 0;
    cudaMemcpy(&flagged, err, 4, cudaMemcpyDeviceToHost);
    const cudaError_t e = cudaDeviceSynchronize();
    printf("\"sms\": %d, \"status\": \"%s\"}\n", sms,
           e != cudaSuccess ? cudaGetErrorString(e) : (flagged ? "a wait timed out" : "ok"));
    return e != cudaSuccess || flagged;
}
