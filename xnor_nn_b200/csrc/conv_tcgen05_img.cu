// Binary convolution on the 5th-generation tensor cores, filters on the M side.
//
//   D[filter][position] += W[tap][filter][channel] * X[position + tap][channel]
//
// Operands are +-1 bytes (0 where a channel, a filter or an image border does not exist), so the
// int32 accumulator is the signed agreement count S of upstream's kernel
// (src/default/bcast_convolution_default.cpp:60-103) exactly: products of absent operands are 0,
// which is upstream's "skip the tap" (:71-72) and its op_c correction (:102) in one.
//
// A tile is 128 filters (UMMA M = the 128 lanes of tensor memory) by R whole output rows of one
// image (UMMA N = R*OW rounded up to 16, at most 256). The activation operand of a filter tap is
// then one 4-D TMA box {channels, OW columns, R rows, 1 image} of the byte tensor, shifted by
// the tap; whatever lies outside the image is filled with zeros by the copy engine, so no
// position is computed that is not an output pixel and no im2col buffer exists. For the 13x13
// AlexNet layers R = 13: a tile is a whole image, and what 32 filters produce for it is one
// contiguous, 128-byte-aligned block of the NCHW result.
//
// One CTA per SM, persistent over its tiles:
//   warp 0      one lane issues the TMA loads of a pipeline stage (a weight tile and an
//               activation box of one filter tap x one channel chunk) into a ring of buffers
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma.kind::i8 (M=128, K=32 per
//               instruction) into one of two accumulators and hands buffers back with
//               tcgen05.commit
//   warps 2-5   epilogue, one warp per 32-lane quadrant of tensor memory = 32 filters: K of the
//               tile's pixels goes to shared memory; tcgen05.ld; scale by alpha[filter] *
//               K[pixel] in upstream's order (:102-103); results are staged in shared memory as
//               [filter][pixel] and leave either as one bulk store (whole-image tiles) or as
//               16-byte-aligned vector stores per filter run. NHWC results are stored straight
//               from registers (a warp store is 32 neighbouring filters of one pixel).
//               The epilogue of a tile runs under the MMAs of the next one (two accumulators).
//
// Tiles are dealt round-robin. When the last round would be less than half full its tiles are
// cut into two row halves, each a tile of its own with a narrower N, so that they occupy twice
// as many SMs for about half as long.
//
// Every wait on an mbarrier is bounded in time: when the bound is hit the kernel records where
// in *error, every role winds down (epilogue warps keep meeting at their named barriers but
// touch nothing), copies in flight are waited for (again bounded), tensor memory is released and
// the kernel returns.
#include <cuda.h>

#include <atomic>

#include "kernels.cuh"
#include "tc_ptx.cuh"

namespace xb200 {

namespace {

using namespace tc;

constexpr int kFilters = 128;       // filters per tile = UMMA M = TMEM lanes
constexpr int kTeam = 2;            // epilogue warps per TMEM lane quadrant (they split the columns)
constexpr int kEpiWarps = 4 * kTeam;
constexpr int kProducerW = 2 + kEpiWarps;  // the warp that loads the weight tiles
constexpr int kThreads = 32 * (kProducerW + 1);
constexpr uint32_t kTmemCols = 512;  // two accumulators of up to 256 columns
constexpr int kMaxStages = 8;
constexpr int kControlBytes = 2304;

struct ImgArgs {
    const float *alpha;
    const float *kmap;   // K per output pixel, or null: box-filter it from amap in the epilogue
    const float *amap;   // mean |x| per input pixel (used when kmap is null)
    float *kmap_out;     // where the epilogue records the K it computed (may be null)
    float *dst;
    int32_t *sums;
    int *error;
    float inv_khw;
    int ih, iw, kh, kw, ph, pw, oh, ow, oc;
    int dst_nhwc;
    // tiles
    int rows, row_blocks, m_blocks;  // output rows per whole tile, tiles per image, filter blocks
    int whole, units;                // whole tiles; work units = whole + 2 * (tiles - whole)
    int half_rows;                   // rows of the first half of a split tile
    // operands
    int kchunk, chunks_per_tap, taps, ocp16;
    uint32_t idesc_full, idesc_half;
    int n_full, n_half;
    uint32_t desc_hi;  // upper 32 bits of the shared-memory matrix descriptors
    uint32_t a_bytes, stage_bytes, tx_full, tx_half;
    int stages;
    // result staging
    int n_staging, ldg;      // buffers; words per filter row when runs are staged one by one
    uint32_t staging_bytes;  // one buffer
    int bulk;                // whole-image tiles whose 32-filter blocks may leave as bulk stores
    unsigned long long wait_ns;
    int drop_commit;  // self-test: CTA 0 leaves out the commit that publishes its first tile
};

struct __align__(16) Control {
    unsigned long long full[kMaxStages];
    unsigned long long empty[kMaxStages];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned long long drain;
    uint32_t tmem_base;
    int abort_flag;
    float kk[2][256];  // K of the tile's pixels, per accumulator
};
static_assert(sizeof(Control) <= kControlBytes, "control block");

struct Tile {
    int n, r0, rows, mt, half;  // image, first output row, rows, filter block, -1 / 0 / 1
};

__device__ __forceinline__ Tile tile_of(const ImgArgs &g, int unit) {
    Tile t;
    int id = unit;
    t.half = -1;
    if (unit >= g.whole) {
        const int j = unit - g.whole;
        id = g.whole + (j >> 1);
        t.half = j & 1;
    }
    t.mt = id % g.m_blocks;
    const int rest = id / g.m_blocks;
    const int rb = rest % g.row_blocks;
    t.n = rest / g.row_blocks;
    t.r0 = rb * g.rows;
    t.rows = g.rows;
    if (t.half == 0) {
        t.rows = g.half_rows;
    } else if (t.half == 1) {
        t.r0 += g.half_rows;
        t.rows = g.rows - g.half_rows;
    }
    return t;
}

__device__ __forceinline__ int rounds_of(const ImgArgs &g) {
    return (g.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
}

// K of output pixel (oh, ow) of image n: box filter of A over the taps inside the image, each
// term scaled by 1/(KH*KW), added in upstream's tap order (src/bcast_calculate_k.cpp:69-85).
__device__ __forceinline__ float box_k(const ImgArgs &g, int n, int oh, int ow) {
    const float *img = g.amap + (long)n * g.ih * g.iw;
    float kk = 0.f;
    for (int i = 0; i < g.kh; i++) {
        const int y = oh - g.ph + i;
        if (y < 0 || y >= g.ih) continue;
        for (int j = 0; j < g.kw; j++) {
            const int x = ow - g.pw + j;
            if (x < 0 || x >= g.iw) continue;
            kk = __fadd_rn(kk, __fmul_rn(__ldg(img + y * g.iw + x), g.inv_khw));
        }
    }
    return kk;
}

// KK = tcgen05.mma instructions per pipeline stage (kchunk / 32).
template <int KK>
__global__ void __launch_bounds__(kThreads, 1)
conv_tcgen05_img_kernel(const __grid_constant__ CUtensorMap map_w,
                        const __grid_constant__ CUtensorMap map_x,
                        const __grid_constant__ CUtensorMap map_xh, const ImgArgs g) {
    extern __shared__ uint8_t smem_raw[];
    // stages need the swizzle atom's alignment (1024 B); staging and the control block follow
    uint8_t *stages = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = stages + (size_t)g.stages * g.stage_bytes;
    Control *ctl = (Control *)(staging + (size_t)g.n_staging * g.staging_bytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &ctl->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; s++) {
            mbar_init(smem_u32(&ctl->full[s]), 2);  // one arrival per producer
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&ctl->acc_full[b]), 1);
            mbar_init(smem_u32(&ctl->acc_empty[b]), 32 * kEpiWarps);
        }
        mbar_init(smem_u32(&ctl->drain), 1);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the descriptors are launch parameters: fetch them while the predecessor still runs
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xh) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    // Everything above touched only this CTA's own shared and tensor memory and the launch
    // parameters. What earlier kernels of the stream produced is read by the TMA producer and
    // the epilogue warps, each after its own dependency_wait(); the MMA issuer reads shared
    // memory only.
    fence_before();
    __syncthreads();
    fence_after();
    // Every CTA of this grid is resident from the start, so a dependent grid may be launched as
    // soon as all of them have got here: its CTAs move in as these exit and set themselves up;
    // they wait for this grid's results themselves.
    dependency_release();
    const uint32_t tmem_base = ctl->tmem_base;

    const int rounds = rounds_of(g);
    const int ksteps = g.taps * g.chunks_per_tap;
    const uint32_t stage0 = smem_u32(stages);

    if (warp == 0 || warp == kProducerW) {
        if (lane == 0) {
            // ---- TMA producers: warp 0 loads the activation boxes, warp kProducerW the weight
            // tiles. Every TMA instruction costs its issuing thread 80-90 cycles and the
            // barrier operations 50-100 each (measured), so the two halves of a stage are
            // issued by two threads; the ring slot's barrier counts both. The next slot's
            // `empty` barrier is tested ahead, as in the MMA issuer. ----
            dependency_wait();
            const bool weights = warp == kProducerW;
            int stage = 0;
            uint32_t phase = 0;
            long issued = 0;  // stage loads issued by this thread
            bool ok = true;
            const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
            const int last_stage = g.stages - 1;
            uint32_t ready = 1;  // the ring starts empty
            uint32_t sa = stage0 + (weights ? 0u : g.a_bytes);
            for (int it = 0; ok && it < rounds; it++) {
                const Tile t = tile_of(g, (int)blockIdx.x + it * (int)gridDim.x);
                const CUtensorMap *mx = t.half >= 0 ? &map_xh : &map_x;
                const uint32_t tx = weights ? g.a_bytes
                                            : (t.half >= 0 ? g.tx_half : g.tx_full) - g.a_bytes;
                int wrow = t.mt * kFilters;  // row of the weight matrix: tap-major
                int y = t.r0 - g.ph, x = -g.pw, kw = 0, c = 0;
                for (int ks = 0; ks < ksteps; ks++) {
                    if (!ready) {
                        const uint32_t ebar = empty0 + 8u * (uint32_t)stage;
                        if (!mbar_try_wait(ebar, phase ^ 1)) {
                            ok = mbar_wait(ebar, phase ^ 1, abort_flag, g.error, 1, g.wait_ns);
                            if (!ok) break;
                        }
                    }
                    const int next = stage == last_stage ? 0 : stage + 1;
                    const uint32_t next_phase = stage == last_stage ? phase ^ 1u : phase;
                    ready = issued + 1 < g.stages ? 1u
                                                  : mbar_test(empty0 + 8u * (uint32_t)next,
                                                              next_phase ^ 1u);
                    const uint32_t bar = full0 + 8u * (uint32_t)stage;
                    mbar_expect_tx(bar, tx);
                    if (weights) tma_load_2d(sa, &map_w, c, wrow, bar);
                    else tma_load_4d(sa, mx, c, x, y, t.n, bar);
                    issued++;
                    sa = next == 0 ? stage0 + (weights ? 0u : g.a_bytes) : sa + g.stage_bytes;
                    stage = next;
                    phase = next_phase;
                    c += g.kchunk;
                    if (c == g.chunks_per_tap * g.kchunk) {  // next filter tap
                        c = 0;
                        wrow += g.ocp16;
                        x++;
                        if (++kw == g.kw) { kw = 0; x = -g.pw; y++; }
                    }
                }
            }
            if (!ok) {
                // Something gave up. Loads already issued still land in this CTA's shared
                // memory: wait for them (bounded) before the CTA may exit.
                for (long j = 0; j < g.stages && j < issued; j++) {
                    const long gi = issued - 1 - j;
                    mbar_wait_quiet(full0 + 8u * (uint32_t)(gi % g.stages),
                                    (uint32_t)((gi / g.stages) & 1), g.wait_ns);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer: a single thread feeds the tensor pipe. Per stage it spends about
            // 25 cycles on each tcgen05.mma and 270 on the tcgen05.commit (measured), so the
            // loop carries nothing else: the next stage's barrier is tested before this stage's
            // instructions are issued and looked at after them. ----
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint64_t hi = (uint64_t)g.desc_hi << 32;
            const uint32_t a_lo0 = ((stage0 >> 4) & 0x3FFF) | (1u << 16);
            const uint32_t b_lo0 = (((stage0 + g.a_bytes) >> 4) & 0x3FFF) | (1u << 16);
            const uint32_t stage_units = g.stage_bytes >> 4;
            const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
            const int last_stage = g.stages - 1;
            uint32_t ready = mbar_test(full0, 0);
            uint32_t desc_off = 0;  // stage * stage_units
            for (int it = 0; ok && it < rounds; it++) {
                const int unit = (int)blockIdx.x + it * (int)gridDim.x;
                const uint32_t idesc = unit >= g.whole ? g.idesc_half : g.idesc_full;
                const int b = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                ok = mbar_wait(smem_u32(&ctl->acc_empty[b]), acc_phase ^ 1, abort_flag, g.error, 2,
                               g.wait_ns);
                if (!ok) break;
                fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * 256);
                uint32_t accumulate = 0;
                for (int ks = 0; ks < ksteps; ks++) {
                    if (!ready) {
                        const uint32_t fbar = full0 + 8u * (uint32_t)stage;
                        if (!mbar_try_wait(fbar, phase)) {
                            ok = mbar_wait(fbar, phase, abort_flag, g.error, 3, g.wait_ns);
                            if (!ok) break;
                        }
                    }
                    const int next = stage == last_stage ? 0 : stage + 1;
                    const uint32_t next_phase = stage == last_stage ? phase ^ 1u : phase;
                    ready = mbar_test(full0 + 8u * (uint32_t)next, next_phase);
                    const uint64_t adesc = hi | (uint64_t)(a_lo0 + desc_off);
                    const uint64_t bdesc = hi | (uint64_t)(b_lo0 + desc_off);
#pragma unroll
                    for (int k = 0; k < KK; k++)
                        mma_i8(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                               k == 0 ? accumulate : 1u);
                    accumulate = 1;
                    commit(empty0 + 8u * (uint32_t)stage);
                    desc_off = next == 0 ? 0u : desc_off + stage_units;
                    stage = next;
                    phase = next_phase;
                }
                if (ok && !(g.drop_commit && it == 0 && blockIdx.x == 0))
                    commit(smem_u32(&ctl->acc_full[b]));
            }
            if (!ok) {
                // Let every MMA already issued finish before tensor memory is released.
                commit(smem_u32(&ctl->drain));
                mbar_wait_quiet(smem_u32(&ctl->drain), 0, g.wait_ns);
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: a team of kTeam warps per quadrant of TMEM lanes = 32 filters; warp
        // `cg` of a team takes every kTeam-th group of 32 columns ----
        dependency_wait();
        const int q = warp & 3, cg = (warp - 2) >> 2, et = threadIdx.x - 64;
        const int e = q;  // teams take turns on the staging buffers in this order
        const int ohw = g.oh * g.ow;
        const bool staged = !g.dst_nhwc || g.sums;
        uint32_t *const out32 = g.sums ? (uint32_t *)g.sums : (uint32_t *)g.dst;
        uint32_t *const sbuf = (uint32_t *)(staging + (size_t)(e % g.n_staging) * g.staging_bytes);
        const long uses = (long)rounds * 4;  // staging-buffer turns of this CTA
        bool live = true;  // false once something gave up: keep the barriers, touch nothing
        for (int it = 0; it < rounds; it++) {
            const Tile t = tile_of(g, (int)blockIdx.x + it * (int)gridDim.x);
            const int b = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int n_cols = t.half >= 0 ? g.n_half : g.n_full;
            const int rows_in = min(t.rows, g.oh - t.r0);
            const int len = rows_in > 0 ? rows_in * g.ow : 0;  // output pixels of the tile
            const long pix0 = (long)t.n * ohw + (long)t.r0 * g.ow;
            if (!g.sums) {
                for (int p = et; p < len; p += 32 * kEpiWarps) {
                    float kk;
                    if (g.kmap) {
                        kk = __ldg(g.kmap + pix0 + p);
                    } else {
                        const int r = p / g.ow;
                        kk = box_k(g, t.n, t.r0 + r, p - r * g.ow);
                        if (g.kmap_out && t.mt == 0) g.kmap_out[pix0 + p] = kk;
                    }
                    ctl->kk[b][p] = kk;
                }
            }
            bar_sync(1, 32 * kEpiWarps);
            if (live)
                live = mbar_wait(smem_u32(&ctl->acc_full[b]), acc_phase, abort_flag, g.error, 4,
                                 g.wait_ns);
            live = __all_sync(0xffffffffu, live);  // tcgen05.ld needs the whole warp
            // my turn on the staging buffer: the warp that used it before has let go of it
            const long use = (long)it * 4 + e;
            if (staged && g.n_staging < 4 && use >= g.n_staging) bar_sync(2 + e, 32 * kTeam + 32);

            const int oc0 = t.mt * kFilters + q * 32, oc = oc0 + lane;
            const float al = (!g.sums && oc < g.oc) ? __ldg(g.alpha + oc) : 0.f;
            // Where this warp's 32 x len results go: the planes of 32 neighbouring filters of one
            // image. When the tile is the whole image they form one contiguous block, staged
            // densely and sent with a single bulk store. Otherwise every filter has a run of its
            // own, staged so that the 16-byte grid of its row in shared memory coincides with the
            // 16-byte grid of global memory (the row is shifted by the run's misalignment).
            uint32_t *const block = out32 + ((long)t.n * g.oc + oc0) * ohw;
            const bool block_mode = g.bulk && t.half < 0 && oc0 + 32 <= g.oc &&
                                    ((uint32_t)(uintptr_t)block & 15u) == 0;
            uint32_t *const run = block + (long)lane * ohw + (long)t.r0 * g.ow;
            const int mis = (int)(((uintptr_t)run >> 2) & 3u);
            uint32_t *const srow_of_lane =
                block_mode ? sbuf + (size_t)lane * ohw : sbuf + (size_t)lane * g.ldg + mis;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * 256);
            if (live) {
                fence_after();
                const float *kk = ctl->kk[b];
                uint32_t *const srow = srow_of_lane;
                for (int c0 = 32 * cg; c0 < n_cols; c0 += 32 * kTeam) {
                    uint32_t v[32];
                    if (c0 + 32 <= n_cols) {
                        ld32(taddr + (uint32_t)c0, v);
                    } else {  // N is a multiple of 16, not always of 32
                        ld16(taddr + (uint32_t)c0, v);
#pragma unroll
                        for (int j = 16; j < 32; j++) v[j] = 0;
                    }
                    wait_ld();
                    if (c0 >= len) continue;
                    if (!g.sums) {
                        // Scale in registers first: K of the 32 pixels comes from shared memory
                        // in one go (the table is padded, entries past `len` are never stored),
                        // so that the stores below do not wait on loads they might alias.
                        float kv[32];
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 k4 = *reinterpret_cast<const float4 *>(kk + c0 + j);
                            kv[j] = k4.x; kv[j + 1] = k4.y; kv[j + 2] = k4.z; kv[j + 3] = k4.w;
                        }
                        // (float)S without the slow conversion pipe: |S| < 2^22, so the integer
                        // lands exactly in the mantissa of 1.5 * 2^23 and one subtraction recovers it
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float sf = __fsub_rn(__uint_as_float(0x4B400000u + v[j]), 12582912.f);
                            v[j] = __float_as_uint(__fmul_rn(__fmul_rn(sf, al), kv[j]));
                        }
                    }
                    if (staged) {
                        if (c0 + 32 <= len) {
#pragma unroll
                            for (int j = 0; j < 32; j++) srow[c0 + j] = v[j];
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (c0 + j < len) srow[c0 + j] = v[j];
                        }
                    } else if (oc < g.oc) {
                        // NHWC: the 32 lanes hold 32 neighbouring filters of one pixel
                        uint32_t *o = out32 + (pix0 + c0) * g.oc + oc;
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (c0 + j < len) o[(long)j * g.oc] = v[j];
                    }
                }
                // the accumulator is in registers / shared memory now: hand it back
                fence_before();
                mbar_arrive(smem_u32(&ctl->acc_empty[b]));
            }
            if (staged) {
                fence_async_smem();
                if (kTeam > 1) bar_sync(6 + q, 32 * kTeam);  // the team's rows are complete
                if (cg == 0 && live && len > 0 && oc0 < g.oc) {
                    if (block_mode) {
                        if (lane == 0) {
                            bulk_store(block, smem_u32(sbuf), (uint32_t)(32 * ohw * 4));
                            bulk_commit();
                            bulk_wait_read();
                        }
                    } else if (oc < g.oc) {
                        // my filter's run: one bulk store for its 16-byte-aligned middle, plain
                        // stores for up to three results on either side
                        int head = (4 - mis) & 3;
                        if (head > len) head = len;
                        const int body = (len - head) & ~3;
                        if (body) {
                            bulk_store(run + head, smem_u32(srow_of_lane + head),
                                       (uint32_t)body * 4u);
                            bulk_commit();
                        }
                        const int done = head + body;
#pragma unroll
                        for (int i = 0; i < 3; i++) {
                            if (i < head) run[i] = srow_of_lane[i];
                            if (done + i < len) run[done + i] = srow_of_lane[done + i];
                        }
                        if (body) bulk_wait_read();
                    }
                    __syncwarp();
                }
                // let the next user of this staging buffer in
                if (cg == 0 && g.n_staging < 4 && use + g.n_staging < uses)
                    bar_arrive(2 + (e + g.n_staging) % 4, 32 * kTeam + 32);
            }
        }
        bulk_wait_all();
    }

    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_free(tmem_base, kTmemCols);
    }
}

}  // namespace

cudaError_t launch_conv_tcgen05_img(const Plan &p, const void *bin_src, const void *bin_w,
                                    const float *alpha, const float *k, const float *a,
                                    float *k_out, float *dst, int32_t *sums, int *error_word,
                                    cudaStream_t s, const ConvSelfTest *test) {
    if (p.mb < 1 || p.img_tiles < 1) return cudaSuccess;
    const uint8_t *x0 = (const uint8_t *)bin_src + (size_t)p.lead * p.icp;  // pixel (0,0) of image 0
    CUtensorMap map_w, map_x, map_xh;
    const uint64_t row = (uint64_t)p.icp;
    const uint32_t half_rows = p.img_half_rows ? (uint32_t)p.img_half_rows : (uint32_t)p.img_rows;
    if (!encode_bytes_2d(&map_w, bin_w, (uint64_t)p.kh * p.kw * p.ocp16, row, (uint32_t)p.kchunk,
                         kFilters) ||
        !encode_bytes_4d(&map_x, x0, row, (uint64_t)p.wp, (uint64_t)p.hp, (uint64_t)p.mb, row,
                         row * p.wp, row * p.wp * p.hp, (uint32_t)p.kchunk, (uint32_t)p.ow,
                         (uint32_t)p.img_rows) ||
        !encode_bytes_4d(&map_xh, x0, row, (uint64_t)p.wp, (uint64_t)p.hp, (uint64_t)p.mb, row,
                         row * p.wp, row * p.wp * p.hp, (uint32_t)p.kchunk, (uint32_t)p.ow,
                         half_rows))
        return cudaErrorNotSupported;

    ImgArgs g;
    g.alpha = alpha; g.kmap = k; g.amap = a; g.kmap_out = k_out; g.dst = dst; g.sums = sums;
    g.error = error_word;
    g.inv_khw = p.inv_khw;
    g.ih = p.ih; g.iw = p.iw; g.kh = p.kh; g.kw = p.kw; g.ph = p.ph; g.pw = p.pw;
    g.oh = p.oh; g.ow = p.ow; g.oc = p.oc;
    g.dst_nhwc = p.dst_nhwc;
    g.rows = p.img_rows; g.row_blocks = p.img_row_blocks; g.m_blocks = p.img_m_blocks;
    g.whole = p.img_whole;
    g.units = p.img_whole + 2 * (p.img_tiles - p.img_whole);
    g.half_rows = p.img_half_rows;
    g.kchunk = p.kchunk; g.chunks_per_tap = p.icp / p.kchunk; g.taps = p.kh * p.kw;
    g.ocp16 = p.ocp16;
    g.n_full = p.img_n;
    g.n_half = p.img_n_half ? p.img_n_half : p.img_n;
    // instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N and M encoded
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kFilters >> 4) << 24);
    g.idesc_full = idesc | ((uint32_t)(g.n_full >> 3) << 17);
    g.idesc_half = idesc | ((uint32_t)(g.n_half >> 3) << 17);
    // matrix descriptor, upper half: stride between 8-row groups (8 * kchunk bytes, in 16-byte
    // units), descriptor version 1, swizzle mode
    const uint32_t sbo = (uint32_t)(8 * p.kchunk) >> 4;
    const uint32_t layout = p.kchunk == 128 ? 2u : p.kchunk == 64 ? 4u : 6u;
    g.desc_hi = sbo | (1u << 14) | (layout << 29);
    g.a_bytes = (uint32_t)(kFilters * p.kchunk);
    g.stage_bytes = ((uint32_t)((kFilters + p.img_n) * p.kchunk) + 1023u) & ~1023u;
    g.tx_full = g.a_bytes + (uint32_t)(p.img_rows * p.ow * p.kchunk);
    g.tx_half = g.a_bytes + half_rows * (uint32_t)(p.ow * p.kchunk);
    g.stages = p.img_stages;
    const bool contiguous = p.img_row_blocks == 1;
    g.ldg = img_staging_row_words(p);
    g.staging_bytes = img_staging_bytes(p);
    g.n_staging = p.img_staging;
    const void *out = sums ? (const void *)sums : (const void *)dst;
    g.bulk = contiguous && !(p.dst_nhwc && !sums) && ((uintptr_t)out & 15) == 0;
    g.wait_ns = test && test->wait_ns ? test->wait_ns : 2000000000ull;
    g.drop_commit = test ? test->drop_commit : 0;

    const int kk = p.kchunk / 32;
    void (*kernel)(CUtensorMap, CUtensorMap, CUtensorMap, ImgArgs) =
        kk == 4 ? conv_tcgen05_img_kernel<4>
        : kk == 2 ? conv_tcgen05_img_kernel<2>
                  : conv_tcgen05_img_kernel<1>;
    size_t smem = 1024 + kControlBytes + (size_t)g.stages * g.stage_bytes +
                  (size_t)g.n_staging * g.staging_bytes;
    // At least 120 KB of shared memory so that one CTA owns the SM and all 512 TMEM columns.
    if (smem < 120 * 1024) smem = 120 * 1024;
    // per device and kernel, once: the opt-in to large dynamic shared memory
    int dev = 0;
    cudaGetDevice(&dev);
    static std::atomic<bool> opted_in[64][3];
    std::atomic<bool> &done = opted_in[dev & 63][kk == 4 ? 0 : kk == 2 ? 1 : 2];
    if (!done.load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(
            kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        done.store(true, std::memory_order_release);
    }
    note_launch();
    return launch_overlapped(kernel, dim3(p.img_grid), dim3(kThreads), smem, s, 1, map_w, map_x,
                             map_xh, g);
}

}  // namespace xb200
