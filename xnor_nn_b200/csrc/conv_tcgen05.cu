// Binary convolution as an implicit GEMM on the 5th-generation tensor cores.
//
// Operands are +-1 bytes (0 where a channel, a filter or an image border does not exist), so the
// int32 accumulator is the signed agreement count S of upstream's kernel
// (src/default/bcast_convolution_default.cpp:60-103) exactly: products of absent operands are 0,
// which is upstream's "skip the tap" (:71-72) and its op_c correction (:102) in one.
//
//   D[position][filter] += A[position + shift(tap)][channel] * B[tap][filter][channel]
//
// The activations live on a zero frame (plan.hpp) on which every filter tap is a constant row
// shift, so the A tile of a tap is a plain 2-D TMA box at a shifted row; no im2col buffer exists.
// Positions on the frame border are computed and dropped by the epilogue.
//
// One CTA per SM, persistent over (position tile, filter tile) pairs:
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor.2d, each CTA fetching its own
//               tiles) into a ring of shared-memory buffers; completion is counted on an
//               mbarrier per buffer
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma.kind::i8 (M=128, N<=256,
//               K=32 per instruction) into one of two accumulators in tensor memory, and
//               tcgen05.commit hands buffers back / accumulators on
//   warp 18     one lane is a second MMA issuer; the two take alternate ring buffers
//   warps 2-17  epilogue: tcgen05.ld the accumulator (a warp owns 32 TMEM lanes = 32 positions
//               and a share of the columns), scale by alpha[filter] * K[position] in upstream's
//               order and store; runs under the next tile's MMAs thanks to the second
//               accumulator
//
// Layers of more than one round of tiles run as clusters of two CTAs on tcgen05 cta_group::2:
// the pair shares a tile of 256 positions x N filters, each CTA loads its own 128 positions and
// half of the filter tile, the leader issues M = 256 instructions for both, and each CTA's
// epilogue drains its own tensor memory. With 128-byte channel chunks a pair loads a position
// tile only once per filter row and chunk, with a halo of the positions that follow it, and the
// taps of the row read that tile at row offsets (producer_halo / mma_role_halo): what bounds the
// kernel is the number of requests an SM can send towards L2, operand reads and result stores
// together.
//
// The epilogue has three forms: floats in NCHW (a warp store is one contiguous run of a filter
// plane), floats in NHWC (a thread owns whole 32-byte sectors and writes them with 256-bit
// stores), and, for chained layers, no floats at all: the sign byte of every result goes into the
// next layer's frame and sum |result| into its mean-|x| map (ChainTarget in kernels.cuh).
//
// Every wait on an mbarrier is bounded in time: when the bound is hit the kernel records where
// in *error, every role winds down, copies in flight are waited for (again bounded), tensor
// memory is released and the kernel returns.
#include <cuda.h>

#include <atomic>
#include <cstddef>
#include <cstdlib>

#include "kernels.cuh"
#include "tc_ptx.cuh"

namespace xb200 {

namespace {

using namespace tc;

constexpr int BM = 128;            // positions per tile = UMMA M = TMEM lanes
constexpr int kMaxStages = 8;       // ring buffers: as many as fit, at most this
constexpr int kEpiWarps = 16;       // epilogue warps: 4 TMEM lane quadrants x column groups
constexpr int kIssuer2Warp = 2 + kEpiWarps;  // the second MMA-issuing thread lives in a warp of its own
constexpr int kThreads = 64 + 32 * kEpiWarps + 32;
constexpr uint32_t kTmemCols = 512;  // two accumulators of up to 256 columns
struct TcArgs {
    const float *alpha;
    const float *kmap;   // K per output pixel, or null: box-filter it from amap in the epilogue
    const float *amap;   // mean |x| per input pixel (used when kmap is null)
    float *kmap_out;     // where the epilogue records the K it computed (may be null)
    float inv_khw;
    int ih, iw, kh;
    float *dst;
    int32_t *sums;
    int *error;
    long q_total;
    int m_tiles, n_tiles, n_tile;
    int kchunk, chunks_per_tap, taps, kw, ph, pw;
    int wp, hp, lead, oh, ow, oc, ocp16;
    uint32_t idesc;
    uint32_t desc_hi;  // upper 32 bits of the shared-memory matrix descriptors
    uint32_t a_bytes, stage_bytes, tx_bytes;
    int dst_nhwc;
    // chained layers: instead of floats the epilogue writes the next layer's packed input
    uint8_t *emit_bin;    // next layer's +-1 byte frame, or null
    float *emit_a;        // next layer's mean-|x| map
    int e_wp, e_hp, e_lead, e_icp;  // the next layer's frame geometry
    float e_inv_ic;       // 1.f / (next layer's channels = this layer's filters)
    int n_inner;          // 1: a CTA works through all filter tiles of a pixel tile in a row
    unsigned long long wait_ns;  // bound of every mbarrier wait
    int drop_commit;      // self-test: CTA 0 leaves out the commit that publishes its first tile
    int issuers;          // threads that issue MMAs: 1, or 2 taking alternate pipeline stages
    int n_stages;         // ring buffers in use
    // Halo mode (pairs, 128-byte chunks, filters at least two taps wide): the position tile of a
    // filter row is loaded once, with the kw - 1 positions that follow it, and serves all kw taps
    // of the row (a tap is a row offset into the tile); the ring then holds filter tiles only.
    int halo;             // 0, or rows of a halo tile (128 + 8)
    int n_a_slots;        // halo tiles in flight
    uint32_t a_slot_bytes, b_ring_off, b_slot_bytes, b_bytes;
    int kk_last;          // MMAs of a tap's last channel chunk: its 32-channel slices that hold
                          // channels at all (the chunk is padded with zero bytes to kchunk)
};

// ---- the kernel --------------------------------------------------------------------------------

constexpr int kAlphaSmem = 2048;  // filters whose alpha is staged in shared memory


struct __align__(16) Control {
    unsigned long long full[kMaxStages];
    unsigned long long empty[kMaxStages];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned long long a_full[4];   // halo mode: a halo tile has landed / has been used up
    unsigned long long a_empty[4];
    unsigned long long started[2];  // two issuers: the tile's first MMA (which overwrites) is out
    unsigned long long drain[2];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float alpha[kAlphaSmem];  // read with 16-byte loads
    float fold[2][4][kEpiWarps / 4][32];  // chained layers: per-warp partial sums of |y|
};
constexpr int kControlBytes = (sizeof(Control) + 1023) / 1024 * 1024;
static_assert(offsetof(Control, alpha) % 16 == 0, "alpha is read as float4");

// Which tile a CTA (PAIR: a pair of CTAs) works on in its it-th round. Default: tiles are dealt
// round-robin with the filter tile as the fast index. n_inner: pixel tiles are dealt round-robin
// and a CTA walks all filter tiles of its pixel tile back to back (so that per-pixel state can be
// carried across them in registers). A pair's tile is two neighbouring pixel tiles, one per CTA.
template <bool PAIR>
struct Deal {
    int unit, units, m_units;
    __device__ __forceinline__ Deal(const TcArgs &g)
        : unit(PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x),
          units(PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x),
          m_units(PAIR ? (g.m_tiles + 1) >> 1 : g.m_tiles) {}
    __device__ __forceinline__ int rounds(const TcArgs &g) const {
        if (g.n_inner) {
            const int mine = (m_units - unit + units - 1) / units;
            return mine > 0 ? mine * g.n_tiles : 0;
        }
        return (m_units * g.n_tiles - unit + units - 1) / units;
    }
    // mt = pixel tile of this CTA
    __device__ __forceinline__ void at(const TcArgs &g, int it, int &mt, int &nt) const {
        int mu;
        if (g.n_inner) {
            const int r = it / g.n_tiles;
            nt = it - r * g.n_tiles;
            mu = unit + r * units;
        } else {
            const int tile = unit + it * units;
            mu = tile / g.n_tiles;
            nt = tile - mu * g.n_tiles;
        }
        mt = PAIR ? 2 * mu + (int)(blockIdx.x & 1) : mu;
    }
};

// ---- epilogue role ---------------------------------------------------------------------------------
// Warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32); several warps share a quadrant and split
// its columns between them.
template <bool PAIR>
__device__ __forceinline__ void epilogue_role(const TcArgs &g, Control *ctl, uint32_t tmem_base,
                                              int warp, int lane, bool alpha_in_smem) {
    volatile int *abort_flag = &ctl->abort_flag;
    const Deal<PAIR> deal(g);
    const int rounds = deal.rounds(g);
    // a pair's accumulators are handed back on the leader's barriers
    const uint32_t acc_empty0 =
        PAIR ? mapa(smem_u32(&ctl->acc_empty[0]), 0) : smem_u32(&ctl->acc_empty[0]);
    // Several warps share a quadrant and split its columns between them.
    const int quad = warp & 3;
    const int cgroup = (warp - 2) >> 2, cgroups = kEpiWarps / 4;
    const int frame = g.hp * g.wp;
    const long ohw = (long)g.oh * g.ow;
    bool ok = true;   // false once a wait ran out somewhere in the CTA
    float run = 0.f;  // chained layers: running sum of |y| over the filter tiles of a pixel
    for (int it = 0; it < rounds; it++) {
        int mt, nt;
        deal.at(g, it, mt, nt);
        const int b = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        const long q = (long)mt * BM + quad * 32 + lane;
        const int n = (int)(q / frame);
        const int rem = (int)(q - (long)n * frame);
        const int oh = rem / g.wp, ow = rem - oh * g.wp;
        const bool valid = q < g.q_total && oh < g.oh && ow < g.ow;
        const int r = oh * g.ow + ow;
        const long pix = (long)n * ohw + r;
        float kk = 0.f;
        if (valid && !g.sums) {
            if (g.kmap) {
                kk = __ldg(g.kmap + pix);
            } else {
                // K = box filter of A over the taps inside the image, each term scaled by
                // 1/(KH*KW), added in upstream's tap order (src/bcast_calculate_k.cpp:69-85)
                const float *img = g.amap + (long)n * g.ih * g.iw;
                for (int i = 0; i < g.kh; i++) {
                    const int y = oh - g.ph + i;
                    if (y < 0 || y >= g.ih) continue;
                    for (int j = 0; j < g.kw; j++) {
                        const int x = ow - g.pw + j;
                        if (x < 0 || x >= g.iw) continue;
                        kk = __fadd_rn(kk, __fmul_rn(__ldg(img + y * g.iw + x), g.inv_khw));
                    }
                }
                if (g.kmap_out && cgroup == 0 && nt == 0) g.kmap_out[pix] = kk;
            }
        }
        const int oc0 = nt * g.n_tile;
        const int n_valid = min(g.n_tile, g.oc - oc0);  // real filters in this tile
        if (ok)
            ok = mbar_wait(smem_u32(&ctl->acc_full[b]), acc_phase, abort_flag, g.error, 4,
                           g.wait_ns);
        ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
        if (!ok) {
            // Given up: touch nothing any more. The chained epilogue's warps of a quadrant meet
            // on a named barrier once per tile; a warp that has given up keeps that appointment
            // so that one that has not (yet) cannot be left waiting there.
            if (g.emit_bin) {
                bar_sync(1 + quad, 32 * (kEpiWarps / 4));
                continue;
            }
            // The NCHW float epilogue's column groups meet three times per tile (all tiles of a
            // CTA but its last): the same appointments are kept here.
            if (!g.sums && !g.dst_nhwc && it + 1 < rounds && g.n_tile == 256) {
                for (int w = 0; w < kEpiWarps / 4 - 1; w++) bar_sync(10, 32 * kEpiWarps);
                continue;
            }
            break;
        }
        fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * g.n_tile);
        if (g.emit_bin) {
            // Chained layers: y = (S * alpha) * K is not stored. alpha and K are never negative,
            // so the sign bit of y is the sign bit of S: it goes straight into the next layer's
            // byte frame (+1 = 0x01, -1 = 0xFF, filters past the last one 0). |y| summed over the
            // filters and divided by their number is that layer's mean-|x| map; K is common to a
            // pixel, so the sum runs over |S| * alpha and is scaled once at the end. A thread
            // owns one pixel and 32 neighbouring filters = 32 contiguous bytes of the frame.
            const float *al = alpha_in_smem ? ctl->alpha + oc0 : g.alpha + oc0;
            uint8_t *row = g.emit_bin +
                           ((long)g.e_lead + ((long)n * g.e_hp + oh) * g.e_wp + ow) * g.e_icp + oc0;
            float part = 0.f;
            for (int c0 = 32 * cgroup; c0 < g.n_tile; c0 += 32 * cgroups) {
                uint32_t v[32];
                const int width = g.n_tile - c0 >= 32 ? 32 : 16;
                if (width == 32) {
                    ld32(taddr + (uint32_t)c0, v);
                } else {
#pragma unroll
                    for (int j = 16; j < 32; j++) v[j] = 0;
                    ld16(taddr + (uint32_t)c0, v);
                }
                wait_ld();
                if (valid) {
                    const int lim = min(n_valid - c0, width);
                    uint32_t w[8];
                    if (alpha_in_smem && lim >= 32) {
                        const float4 *a4 = reinterpret_cast<const float4 *>(al + c0);
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 a = a4[j >> 2];
                            part = fmaf(fabsf((float)(int)v[j]), a.x, part);
                            part = fmaf(fabsf((float)(int)v[j + 1]), a.y, part);
                            part = fmaf(fabsf((float)(int)v[j + 2]), a.z, part);
                            part = fmaf(fabsf((float)(int)v[j + 3]), a.w, part);
                            // byte 3 of each count, sign-replicated: 0xFF where S < 0, else 0
                            const uint32_t lo = __byte_perm(v[j], v[j + 1], 0x00FB);
                            const uint32_t hi = __byte_perm(v[j + 2], v[j + 3], 0x00FB);
                            w[j >> 2] = __byte_perm(lo, hi, 0x5410) | 0x01010101u;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            uint32_t word = 0;
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                if (j + i < lim) {
                                    part = fmaf(fabsf((float)(int)v[j + i]), al[c0 + j + i], part);
                                    word |= ((v[j + i] >> 31) ? 0xFFu : 0x01u) << (8 * i);
                                }
                            }
                            w[j >> 2] = word;
                        }
                    }
                    if (width == 32 && oc0 + c0 + 32 <= g.e_icp && ((oc0 + c0) & 31) == 0) {
                        // one whole 32-byte sector per thread in a single store
                        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                     ::"l"(row + c0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                                       "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                                     : "memory");
                    } else {
                        if (oc0 + c0 + 16 <= g.e_icp)
                            *reinterpret_cast<uint4 *>(row + c0) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        if (width == 32 && oc0 + c0 + 32 <= g.e_icp)
                            *reinterpret_cast<uint4 *>(row + c0 + 16) =
                                make_uint4(w[4], w[5], w[6], w[7]);
                    }
                }
            }
            // Fold the column groups' partial sums in a fixed order (group 0, 1, 2, 3, then the
            // next filter tile), so the map is reproducible; the four warps of a lane quadrant
            // meet on a named barrier of their own.
            ctl->fold[it & 1][quad][cgroup][lane] = part;
            bar_sync(1 + quad, 32 * (kEpiWarps / 4));
            if (cgroup == 0) {
                if (nt == 0) run = 0.f;
#pragma unroll
                for (int c = 0; c < kEpiWarps / 4; c++)
                    run = __fadd_rn(run, ctl->fold[it & 1][quad][c][lane]);
                if (nt == g.n_tiles - 1 && valid)
                    g.emit_a[pix] = __fmul_rn(__fmul_rn(run, kk), g.e_inv_ic);
            }
        } else if (!g.sums && !g.dst_nhwc) {
            // NCHW floats: for one filter the 32 lanes hold 32 neighbouring pixels, so a
            // store instruction writes one contiguous run.
            float *out = g.dst + ((long)n * g.oc + oc0) * ohw + r;
            const float *al = alpha_in_smem ? ctl->alpha + oc0 : g.alpha + oc0;
            // Except for a CTA's last tile the four column groups store one after the other
            // (three meetings of all epilogue warps per tile, column group c stores between the
            // c-th and the next): the stores of a tile then leave the SM over about twice the
            // time, which leaves the SM's request port more room for the next tile's operand
            // loads (conv4 32.7 -> 31.6 us, VGG 78.6 -> 76.9). Only for tiles of 256 filters: with
            // narrower ones (conv3, N = 192) a tile's MMAs are over sooner than its epilogue
            // spread out like this, and the whole step got slower (55.1 -> 57.7 us).
            const bool paced = it + 1 < rounds && g.n_tile == 256;
            if (paced) for (int w = 0; w < cgroup; w++) bar_sync(10, 32 * kEpiWarps);
            for (int c0 = 32 * cgroup; c0 < g.n_tile; c0 += 32 * cgroups) {
                uint32_t v[32];
                if (c0 + 32 <= g.n_tile) {
                    ld32(taddr + (uint32_t)c0, v);
                } else {  // N is a multiple of 16, not always of 32
                    ld16(taddr + (uint32_t)c0, v);
                }
                wait_ld();
                if (valid) {
                    const int lim = n_valid - c0;
                    float *o = out + (long)c0 * ohw;
                    if (alpha_in_smem && lim >= 32) {
                        // full group: alpha by 16-byte shared loads, one running pointer
                        const float4 *a4 = reinterpret_cast<const float4 *>(al + c0);
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 a = a4[j >> 2];
                            // streaming stores: the result is not read again by this library,
                            // and lines that leave L2 while this kernel runs (which needs little
                            // of HBM) do not have to leave it under the next, bandwidth-bound pass
                            __stcs(o, __fmul_rn(__fmul_rn((float)(int)v[j], a.x), kk));
                            __stcs(o + ohw, __fmul_rn(__fmul_rn((float)(int)v[j + 1], a.y), kk));
                            __stcs(o + 2 * ohw, __fmul_rn(__fmul_rn((float)(int)v[j + 2], a.z), kk));
                            __stcs(o + 3 * ohw, __fmul_rn(__fmul_rn((float)(int)v[j + 3], a.w), kk));
                            o += 4 * ohw;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < lim)
                                __stcs(o + (long)j * ohw,
                                       __fmul_rn(__fmul_rn((float)(int)v[j], al[c0 + j]), kk));
                    }
                }
            }
            if (paced) for (int w = cgroup; w < kEpiWarps / 4 - 1; w++) bar_sync(10, 32 * kEpiWarps);
        } else if (!g.sums && g.dst_nhwc && (g.oc & 3) == 0) {
            // NHWC floats: a thread owns one pixel and 16 neighbouring filters at a time, which
            // are contiguous in the result: four 16-byte stores.
            float *out = g.dst + pix * g.oc + oc0;
            const float *al = alpha_in_smem ? ctl->alpha + oc0 : g.alpha + oc0;
            // 256-bit stores need 32-byte alignment: rows and tiles that are multiples of 8
            // floats on a result buffer aligned likewise
            const bool wide = (g.oc & 7) == 0 && (oc0 & 7) == 0 && ((uintptr_t)g.dst & 31) == 0;
            for (int c0 = 16 * cgroup; c0 < g.n_tile; c0 += 16 * cgroups) {
                uint32_t v[16];
                ld16(taddr + (uint32_t)c0, v);
                wait_ld();
                if (valid && wide && c0 + 16 <= n_valid) {
                    // 16 results = two whole 32-byte sectors, one 256-bit store each
                    float x[16];
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        x[j] = __fmul_rn(__fmul_rn((float)(int)v[j], al[c0 + j]), kk);
#pragma unroll
                    for (int h = 0; h < 16; h += 8)
                        asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                     ::"l"(out + c0 + h), "f"(x[h]), "f"(x[h + 1]), "f"(x[h + 2]),
                                       "f"(x[h + 3]), "f"(x[h + 4]), "f"(x[h + 5]), "f"(x[h + 6]),
                                       "f"(x[h + 7])
                                     : "memory");
                } else if (valid) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        if (c0 + j >= n_valid) break;  // oc and n_valid are multiples of 4
                        float4 x;
                        x.x = __fmul_rn(__fmul_rn((float)(int)v[j], al[c0 + j]), kk);
                        x.y = __fmul_rn(__fmul_rn((float)(int)v[j + 1], al[c0 + j + 1]), kk);
                        x.z = __fmul_rn(__fmul_rn((float)(int)v[j + 2], al[c0 + j + 2]), kk);
                        x.w = __fmul_rn(__fmul_rn((float)(int)v[j + 3], al[c0 + j + 3]), kk);
                        *reinterpret_cast<float4 *>(out + c0 + j) = x;
                    }
                }
            }
        } else {
            for (int c0 = 16 * cgroup; c0 < g.n_tile; c0 += 16 * cgroups) {
                uint32_t v[16];
                ld16(taddr + (uint32_t)c0, v);
                wait_ld();
                if (valid) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int oc = oc0 + c0 + j;
                        if (oc >= g.oc) continue;
                        if (g.sums) {
                            g.sums[((long)n * g.oc + oc) * ohw + r] = (int)v[j];
                        } else {
                            const float x =
                                __fmul_rn(__fmul_rn((float)(int)v[j], __ldg(g.alpha + oc)), kk);
                            if (g.dst_nhwc) g.dst[pix * g.oc + oc] = x;
                            else g.dst[((long)n * g.oc + oc) * ohw + r] = x;
                        }
                    }
                }
            }
        }
        fence_before();
        if (PAIR) {
            // one arrival per warp: tcgen05.wait::ld is warp-wide, so every lane's reads are done
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8u * (uint32_t)b);
        } else {
            mbar_arrive(acc_empty0 + 8u * (uint32_t)b);
        }
    }
}

// ---- MMA issuer role -----------------------------------------------------------------------------
// One thread feeds the tensor pipe; the instructions of a pipeline stage (KK tcgen05.mma and the
// tcgen05.commit that hands the stage back) cost that thread more cycles than the pipe needs for
// them unless N is 256. With two issuers the stages are dealt alternately (issuer i takes stages
// i, i+2, ... of the running stage sequence, which continues across tiles), each commits its own
// stages, and both commit to the accumulator's barrier (count 2) after their last stage of a
// tile: a commit covers the MMAs of the committing thread only. The sum is over integers, so the
// order in which the two threads' MMAs reach the pipe does not matter, except for the tile's
// first instruction, which overwrites the accumulator: its issuer waits for the epilogue to have
// drained the accumulator, and the other issuer waits for it (started[]).
template <int KK, bool PAIR>
__device__ __forceinline__ void mma_role(const TcArgs &g, Control *ctl, uint32_t tmem_base,
                                         uint32_t stage0, int who) {
    volatile int *abort_flag = &ctl->abort_flag;
    const int rounds = Deal<PAIR>(g).rounds(g);
    if (rounds == 0) return;
    const int ksteps = g.taps * g.chunks_per_tap;  // >= g.issuers (the launcher sees to it)
    const int n_iss = g.issuers;
    const uint64_t hi = (uint64_t)g.desc_hi << 32;
    const uint32_t a_lo0 = ((stage0 >> 4) & 0x3FFF) | (1u << 16);
    const uint32_t b_lo0 = (((stage0 + g.a_bytes) >> 4) & 0x3FFF) | (1u << 16);
    const uint32_t stage_units = g.stage_bytes >> 4;
    const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
    const int n_stages = g.n_stages;  // >= g.issuers
    int it = 0, ks = who, stage = who;
    // position of this thread's current stage among the chunks of its tap
    int chunk = who % g.chunks_per_tap;
    const int chunk_step = n_iss % g.chunks_per_tap;
    uint32_t phase = 0;
    bool ok = true, entered = false;
    for (;;) {
        const int b = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!entered) {
            if (ks == 0)
                ok = mbar_wait(smem_u32(&ctl->acc_empty[b]), acc_phase ^ 1, abort_flag, g.error, 2,
                               g.wait_ns);
            else if (n_iss > 1)
                ok = mbar_wait(smem_u32(&ctl->started[b]), acc_phase, abort_flag, g.error, 6,
                               g.wait_ns);
            if (!ok) break;
            fence_after();
            entered = true;
        }
        const uint32_t fbar = full0 + 8u * (uint32_t)stage;
        if (!mbar_try_wait(fbar, phase)) {
            ok = mbar_wait(fbar, phase, abort_flag, g.error, 3, g.wait_ns);
            if (!ok) break;
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * g.n_tile);
        const uint32_t desc_off = (uint32_t)stage * stage_units;
        const uint64_t adesc = hi | (uint64_t)(a_lo0 + desc_off);
        const uint64_t bdesc = hi | (uint64_t)(b_lo0 + desc_off);
        // slices of zero padding behind the last channel are not multiplied
        const int kk = chunk == g.chunks_per_tap - 1 ? g.kk_last : KK;
#pragma unroll
        for (int k = 0; k < KK; k++) {
            if (k < kk) {
                if (PAIR)
                    mma_i8_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k),
                                g.idesc, (k == 0 && ks == 0) ? 0u : 1u);
                else
                    mma_i8(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), g.idesc,
                           (k == 0 && ks == 0) ? 0u : 1u);
            }
        }
        if (PAIR) commit_pair(empty0 + 8u * (uint32_t)stage);  // frees the stage in both CTAs
        else commit(empty0 + 8u * (uint32_t)stage);
        if (n_iss > 1 && ks == 0) {
            fence_before();
            mbar_arrive(smem_u32(&ctl->started[b]));
        }
        stage += n_iss;
        if (stage >= n_stages) { stage -= n_stages; phase ^= 1u; }
        chunk += chunk_step;
        if (chunk >= g.chunks_per_tap) chunk -= g.chunks_per_tap;
        ks += n_iss;
        if (ks >= ksteps) {  // this thread's share of the tile is issued
            ks -= ksteps;
            if (!(g.drop_commit && it == 0 && blockIdx.x == 0)) {
                if (PAIR) commit_pair(smem_u32(&ctl->acc_full[b]));
                else commit(smem_u32(&ctl->acc_full[b]));
            }
            entered = false;
            if (++it >= rounds) break;
        }
    }
    if (!ok) {
        // Let every MMA this thread has issued finish before tensor memory is released.
        if (PAIR) commit_pair(smem_u32(&ctl->drain[who]));
        else commit(smem_u32(&ctl->drain[who]));
        mbar_wait_quiet(smem_u32(&ctl->drain[who]), 0, g.wait_ns);
    }
}

// ---- halo mode: producer and MMA issuers -----------------------------------------------------------
// Step order inside a tile: filter row kh, channel chunk, filter column kw (the sums are integers:
// any order gives the same result). A group = the kw steps of one (kh, chunk): one halo tile of
// g.halo positions in slot G % n_a_slots (G counts groups across tiles), kw filter tiles in
// consecutive slots of the filter ring. A descriptor that starts r rows into a 128-byte-swizzled
// tile reads rows r .. r + 127 of it (the swizzle is a function of the shared-memory address), so
// tap kw of the group is the halo tile's descriptor advanced by kw rows.
template <bool PAIR>
__device__ __forceinline__ void producer_halo(const TcArgs &g, Control *ctl,
                                              const CUtensorMap *map_a, const CUtensorMap *map_b,
                                              uint32_t stage0, uint32_t rank) {
    volatile int *abort_flag = &ctl->abort_flag;
    const Deal<PAIR> deal(g);
    const int rounds = deal.rounds(g);
    const uint32_t full_l = smem_u32(&ctl->full[0]), afull_l = smem_u32(&ctl->a_full[0]);
    // a pair counts both CTAs' bytes on the leader's barriers
    const uint32_t full0 = PAIR && rank != 0 ? mapa(full_l, 0) : full_l;
    const uint32_t afull0 = PAIR && rank != 0 ? mapa(afull_l, 0) : afull_l;
    const uint32_t empty0 = smem_u32(&ctl->empty[0]), aempty0 = smem_u32(&ctl->a_empty[0]);
    const int b_rows = PAIR ? g.n_tile >> 1 : g.n_tile;
    const uint32_t mult = PAIR ? 2u : 1u;
    const uint32_t a_bytes = (uint32_t)g.halo * (uint32_t)g.kchunk;
    int sb = 0, sa = 0;
    uint32_t pb = 0, pa = 0;
    uint32_t armed_b = 0, parity_b = 0, armed_a = 0, parity_a = 0;
    bool ok = true;
    for (int it = 0; ok && it < rounds; it++) {
        int mt, nt;
        deal.at(g, it, mt, nt);
        const int row0 = g.lead + mt * BM - g.ph * g.wp - g.pw;  // tap (0,0)
        const int brow0 = nt * g.n_tile + (int)rank * b_rows;
        for (int kh = 0; ok && kh < g.kh; kh++) {
            for (int chunk = 0; ok && chunk < g.chunks_per_tap; chunk++) {
                const uint32_t aebar = aempty0 + 8u * (uint32_t)sa;
                if (!mbar_try_wait(aebar, pa ^ 1)) {
                    ok = mbar_wait(aebar, pa ^ 1, abort_flag, g.error, 8, g.wait_ns);
                    if (!ok) break;
                }
                const uint32_t abar = afull0 + 8u * (uint32_t)sa;
                if (!PAIR || rank == 0) mbar_expect_tx(abar, mult * a_bytes);  // abar is local here
                const uint32_t adst = stage0 + (uint32_t)sa * g.a_slot_bytes;
                if (PAIR) tma_load_2d_pair(adst, map_a, chunk * g.kchunk, row0 + kh * g.wp, abar);
                else tma_load_2d(adst, map_a, chunk * g.kchunk, row0 + kh * g.wp, abar);
                armed_a |= 1u << sa;
                parity_a = (parity_a & ~(1u << sa)) | (pa << sa);
                if (++sa == g.n_a_slots) { sa = 0; pa ^= 1; }
                int brow = brow0 + kh * g.kw * g.ocp16;
                for (int kw = 0; kw < g.kw; kw++, brow += g.ocp16) {
                    const uint32_t ebar = empty0 + 8u * (uint32_t)sb;
                    if (!mbar_try_wait(ebar, pb ^ 1)) {
                        ok = mbar_wait(ebar, pb ^ 1, abort_flag, g.error, 1, g.wait_ns);
                        if (!ok) break;
                    }
                    const uint32_t bar = full0 + 8u * (uint32_t)sb;
                    if (!PAIR || rank == 0) mbar_expect_tx(bar, mult * g.b_bytes);
                    const uint32_t bdst = stage0 + g.b_ring_off + (uint32_t)sb * g.b_slot_bytes;
                    if (PAIR) tma_load_2d_pair(bdst, map_b, chunk * g.kchunk, brow, bar);
                    else tma_load_2d(bdst, map_b, chunk * g.kchunk, brow, bar);
                    armed_b |= 1u << sb;
                    parity_b = (parity_b & ~(1u << sb)) | (pb << sb);
                    if (++sb == g.n_stages) { sb = 0; pb ^= 1; }
                }
            }
        }
    }
    if (!ok && rank == 0) {
        // Something gave up. Loads already issued still land in this CTA's shared memory: wait
        // for them (bounded) before the CTA may exit.
        for (int s = 0; s < g.n_stages; s++)
            if (armed_b & (1u << s))
                mbar_wait_quiet(full_l + 8u * (uint32_t)s, (parity_b >> s) & 1u, g.wait_ns);
        for (int s = 0; s < g.n_a_slots; s++)
            if (armed_a & (1u << s))
                mbar_wait_quiet(afull_l + 8u * (uint32_t)s, (parity_a >> s) & 1u, g.wait_ns);
    }
}

template <int KK, bool PAIR>
__device__ __forceinline__ void mma_role_halo(const TcArgs &g, Control *ctl, uint32_t tmem_base,
                                              uint32_t stage0, int who) {
    volatile int *abort_flag = &ctl->abort_flag;
    const int rounds = Deal<PAIR>(g).rounds(g);
    if (rounds == 0) return;
    const int ksteps = g.taps * g.chunks_per_tap;  // >= g.issuers; a multiple of g.kw
    const int n_iss = g.issuers, kwn = g.kw;
    const uint64_t hi = (uint64_t)g.desc_hi << 32;
    const uint32_t a_lo0 = ((stage0 >> 4) & 0x3FFF) | (1u << 16);
    const uint32_t b_lo0 = (((stage0 + g.b_ring_off) >> 4) & 0x3FFF) | (1u << 16);
    const uint32_t a_units = g.a_slot_bytes >> 4, b_units = g.b_slot_bytes >> 4;
    const uint32_t row_units = (uint32_t)g.kchunk >> 4;  // one position further
    const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
    const uint32_t afull0 = smem_u32(&ctl->a_full[0]), aempty0 = smem_u32(&ctl->a_empty[0]);
    int it = 0, ks = who;
    int sb = who % g.n_stages;
    uint32_t pb = 0;
    // the group of this thread's current step: its column kw, its halo slot
    int kw = who % kwn, sa = (who / kwn) % g.n_a_slots;
    uint32_t pa = ((who / kwn) / g.n_a_slots) & 1u;
    int chunk = (who / kwn) % g.chunks_per_tap;  // groups walk the chunks, then the filter rows
    bool ok = true, entered = false, a_seen = false;
    for (;;) {
        const int b = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!entered) {
            if (ks == 0)
                ok = mbar_wait(smem_u32(&ctl->acc_empty[b]), acc_phase ^ 1, abort_flag, g.error, 2,
                               g.wait_ns);
            else if (n_iss > 1)
                ok = mbar_wait(smem_u32(&ctl->started[b]), acc_phase, abort_flag, g.error, 6,
                               g.wait_ns);
            if (!ok) break;
            fence_after();
            entered = true;
        }
        if (!a_seen) {  // first step of this thread in the group: the halo tile must have landed
            const uint32_t abar = afull0 + 8u * (uint32_t)sa;
            if (!mbar_try_wait(abar, pa)) {
                ok = mbar_wait(abar, pa, abort_flag, g.error, 9, g.wait_ns);
                if (!ok) break;
            }
            a_seen = true;
        }
        const uint32_t fbar = full0 + 8u * (uint32_t)sb;
        if (!mbar_try_wait(fbar, pb)) {
            ok = mbar_wait(fbar, pb, abort_flag, g.error, 3, g.wait_ns);
            if (!ok) break;
        }
        fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * g.n_tile);
        const uint64_t adesc =
            hi | (uint64_t)(a_lo0 + (uint32_t)sa * a_units + (uint32_t)kw * row_units);
        const uint64_t bdesc = hi | (uint64_t)(b_lo0 + (uint32_t)sb * b_units);
        const int kk = chunk == g.chunks_per_tap - 1 ? g.kk_last : KK;
#pragma unroll
        for (int k = 0; k < KK; k++) {
            if (k < kk) {
                if (PAIR)
                    mma_i8_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k),
                                g.idesc, (k == 0 && ks == 0) ? 0u : 1u);
                else
                    mma_i8(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), g.idesc,
                           (k == 0 && ks == 0) ? 0u : 1u);
            }
        }
        if (PAIR) commit_pair(empty0 + 8u * (uint32_t)sb);
        else commit(empty0 + 8u * (uint32_t)sb);
        if (n_iss > 1 && ks == 0) {
            fence_before();
            mbar_arrive(smem_u32(&ctl->started[b]));
        }
        sb += n_iss;
        if (sb >= g.n_stages) { sb -= g.n_stages; pb ^= 1u; }
        kw += n_iss;
        if (kw >= kwn) {
            // this thread's last step of the group is issued: its reads of the halo tile are
            // covered by this commit (both issuers commit: the barrier counts them)
            if (PAIR) commit_pair(aempty0 + 8u * (uint32_t)sa);
            else commit(aempty0 + 8u * (uint32_t)sa);
            do {
                kw -= kwn;
                if (++sa == g.n_a_slots) { sa = 0; pa ^= 1u; }
                if (++chunk == g.chunks_per_tap) chunk = 0;
            } while (kw >= kwn);
            a_seen = false;
        }
        ks += n_iss;
        if (ks >= ksteps) {  // this thread's share of the tile is issued
            ks -= ksteps;
            if (!(g.drop_commit && it == 0 && blockIdx.x == 0)) {
                if (PAIR) commit_pair(smem_u32(&ctl->acc_full[b]));
                else commit(smem_u32(&ctl->acc_full[b]));
            }
            entered = false;
            if (++it >= rounds) break;
        }
    }
    if (!ok) {
        if (PAIR) commit_pair(smem_u32(&ctl->drain[who]));
        else commit(smem_u32(&ctl->drain[who]));
        mbar_wait_quiet(smem_u32(&ctl->drain[who]), 0, g.wait_ns);
    }
}

// KK = tcgen05.mma instructions per pipeline stage (kchunk / 32).
// PAIR: the grid is made of clusters of two CTAs that share tiles of 256 positions x N filters
// (tcgen05 cta_group::2). Each CTA loads its own 128 positions and its half of the filter tile,
// the leader (rank 0) issues one M = 256 instruction for both, and each CTA's epilogue drains its
// own tensor memory. A stage is a third smaller per CTA that way (32 KB instead of 48 KB at
// N = 256), which is what the kernel is short of: at one stage per 512 cycles a single CTA pulls
// 94 B/clk from L2, four fifths of what the SM's port delivers.
template <int KK, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
conv_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, const TcArgs g) {
    extern __shared__ uint8_t smem_raw[];
    // stages need the swizzle atom's alignment (1024 B); the control block sits in front
    uint8_t *base = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Control *ctl = (Control *)base;
    uint8_t *stages = base + kControlBytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &ctl->abort_flag;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < g.n_stages; s++) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int a = 0; a < 4; a++) {
            mbar_init(smem_u32(&ctl->a_full[a]), 1);
            mbar_init(smem_u32(&ctl->a_empty[a]), (uint32_t)g.issuers);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&ctl->acc_full[b]), (uint32_t)g.issuers);
            // single CTA: one arrival per epilogue thread; pair: one per epilogue warp of both
            mbar_init(smem_u32(&ctl->acc_empty[b]), PAIR ? 2 * kEpiWarps : 32 * kEpiWarps);
            mbar_init(smem_u32(&ctl->started[b]), 1);
            mbar_init(smem_u32(&ctl->drain[b]), 1);
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the descriptors are launch parameters: fetch them while the predecessor still runs
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) {
        // Each CTA allocates all of its own tensor memory, so the accumulators sit at the same
        // address in both CTAs of a pair.
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    }
    // Everything above touched only this CTA's own shared and tensor memory and the launch
    // parameters. What earlier kernels of the stream produced is read by the TMA producer and
    // the epilogue warps, each after its own dependency_wait(); the MMA issuer reads shared
    // memory only.
    const bool alpha_in_smem = g.ocp16 <= kAlphaSmem;
    fence_before();
    __syncthreads();
    if (PAIR) {  // the partner's barriers exist before anything is sent to them
        cluster_arrive();
        cluster_wait();
    }
    fence_after();
    // Every CTA of this grid is resident from the start, so a dependent grid may be launched as
    // soon as all of them have got here: its CTAs move in as these exit (SMs with one tile fewer
    // exit a round early) and set themselves up; they wait for this grid's results themselves.
    dependency_release();
    const uint32_t tmem_base = ctl->tmem_base;

    const Deal<PAIR> deal(g);
    const int rounds = deal.rounds(g);
    const int ksteps = g.taps * g.chunks_per_tap;
    const uint32_t stage0 = smem_u32(stages);

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            dependency_wait();
            if (g.halo) {
                producer_halo<PAIR>(g, ctl, &map_a, &map_b, stage0, rank);
            } else {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;  // bit s: stage s holds a load nobody is known to have consumed
            uint32_t armed_parity = 0;
            bool ok = true;
            // a pair counts both CTAs' bytes on the leader's barrier
            const uint32_t full_local = smem_u32(&ctl->full[0]);
            const uint32_t full0 = PAIR && rank != 0 ? mapa(full_local, 0) : full_local;
            const int b_rows = PAIR ? g.n_tile >> 1 : g.n_tile;  // filter rows this CTA loads
            for (int it = 0; ok && it < rounds; it++) {
                int mt, nt;
                deal.at(g, it, mt, nt);
                int row = g.lead + mt * BM - g.ph * g.wp - g.pw;  // tap (0,0)
                int brow = nt * g.n_tile + (int)rank * b_rows;
                int kw = 0, chunk = 0;
                for (int ks = 0; ks < ksteps; ks++) {
                    const uint32_t ebar = smem_u32(&ctl->empty[stage]);
                    if (!mbar_try_wait(ebar, phase ^ 1)) {
                        ok = mbar_wait(ebar, phase ^ 1, abort_flag, g.error, 1, g.wait_ns);
                        if (!ok) break;
                    }
                    armed &= ~(1u << stage);
                    const uint32_t bar = full0 + 8u * (uint32_t)stage;
                    const uint32_t sa = stage0 + (uint32_t)stage * g.stage_bytes;
                    if (PAIR) {
                        if (rank == 0) mbar_expect_tx(bar, 2u * g.tx_bytes);  // bar is local here
                        tma_load_2d_pair(sa, &map_a, chunk * g.kchunk, row, bar);
                        tma_load_2d_pair(sa + g.a_bytes, &map_b, chunk * g.kchunk, brow, bar);
                    } else {
                        mbar_expect_tx(bar, g.tx_bytes);
                        tma_load_2d(sa, &map_a, chunk * g.kchunk, row, bar);
                        tma_load_2d(sa + g.a_bytes, &map_b, chunk * g.kchunk, brow, bar);
                    }
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == g.n_stages) { stage = 0; phase ^= 1; }
                    if (++chunk == g.chunks_per_tap) {  // next filter tap
                        chunk = 0;
                        brow += g.ocp16;
                        if (++kw == g.kw) { kw = 0; row += g.wp - (g.kw - 1); }
                        else row += 1;
                    }
                }
            }
            if (!ok && rank == 0) {
                // Something gave up. Loads already issued still land in this CTA's shared
                // memory: wait for them (bounded) before the CTA may exit. (The partner of a
                // pair cannot wait on the leader's barrier; it stays until the leader has got
                // through this and both have met at the cluster barrier below.)
                for (int s = 0; s < g.n_stages; s++)
                    if (armed & (1u << s)) {
                        mbar_wait_quiet(smem_u32(&ctl->full[s]), (armed_parity >> s) & 1u,
                                        g.wait_ns);
                    }
            }
            }
        }
    } else if (warp == 1 || warp == kIssuer2Warp) {
        const int who = warp == 1 ? 0 : 1;
        if (lane == 0 && who < g.issuers && rank == 0) {
            if (g.halo) mma_role_halo<KK, PAIR>(g, ctl, tmem_base, stage0, who);
            else mma_role<KK, PAIR>(g, ctl, tmem_base, stage0, who);
        }
        __syncwarp();
    } else {
        // ---- epilogue warps: stage alpha among themselves, then drain accumulators ----
        dependency_wait();
        if (alpha_in_smem) {
            for (int i = threadIdx.x - 64; i < g.ocp16; i += 32 * kEpiWarps)
                ctl->alpha[i] = i < g.oc ? __ldg(g.alpha + i) : 0.f;
            bar_sync(5, 32 * kEpiWarps);
        }
        epilogue_role<PAIR>(g, ctl, tmem_base, warp, lane, alpha_in_smem);
    }

    fence_before();
    __syncthreads();
    if (PAIR) {
        // Neither CTA leaves while the other may still read its shared or tensor memory or
        // signal its barriers.
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        fence_after();
        tmem_free(tmem_base, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------

}  // namespace

cudaError_t launch_conv_tcgen05(const Plan &p, const void *bin_src, const void *bin_w,
                                const float *alpha, const float *k, const float *a, float *k_out,
                                float *dst, int32_t *sums, int *error_word, cudaStream_t s,
                                const ChainTarget *next, const ConvSelfTest *test) {
    if (p.q_total == 0) return cudaSuccess;
    const int m_tiles = (int)((p.q_total + BM - 1) / BM);
    int dev = 0;
    cudaGetDevice(&dev);
    static std::atomic<int> sm_count[64], pair_count[64];
    const int d = dev & 63;
    int sms = sm_count[d].load(std::memory_order_relaxed);
    if (!sms) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        sm_count[d].store(sms, std::memory_order_relaxed);
    }
    // CTA pairs when the layer is more than one round of tiles (measured on AlexNet conv4: 35.0
    // against 36.9 us at 256 images, 24.3 against 24.9 at 128; with a single round the pair's
    // longer hand-shakes cost more than its lighter loads save: 15.6 against 14.7 us at 64
    // images). Floats or sums out only (the chained epilogue carries per-pixel state across the
    // filter tiles of one CTA), and a filter tile that splits into two UMMA-sized halves.
    const bool pair = !next && p.n_tile % 32 == 0 && m_tiles >= 2 &&
                      (long)m_tiles * (p.ocp16 / p.n_tile) > sms;
    const int b_rows = pair ? p.n_tile / 2 : p.n_tile;  // filter rows a CTA loads per stage
    TcArgs g;
    g.alpha = alpha; g.kmap = k; g.amap = a; g.kmap_out = k_out; g.dst = dst; g.sums = sums;
    g.error = error_word;
    g.inv_khw = p.inv_khw; g.ih = p.ih; g.iw = p.iw; g.kh = p.kh;
    g.q_total = p.q_total;
    g.m_tiles = m_tiles;
    g.n_tiles = p.ocp16 / p.n_tile;
    g.n_tile = p.n_tile;
    g.kchunk = p.kchunk; g.chunks_per_tap = p.icp / p.kchunk; g.taps = p.kh * p.kw;
    g.kw = p.kw; g.ph = p.ph; g.pw = p.pw; g.wp = p.wp; g.hp = p.hp; g.lead = p.lead;
    g.oh = p.oh; g.ow = p.ow; g.oc = p.oc; g.ocp16 = p.ocp16;
    g.dst_nhwc = p.dst_nhwc;
    g.emit_bin = nullptr; g.emit_a = nullptr; g.n_inner = 0;
    g.wait_ns = test && test->wait_ns ? test->wait_ns : 2000000000ull;
    g.drop_commit = test ? test->drop_commit : 0;
    g.e_wp = g.e_hp = g.e_lead = g.e_icp = 0; g.e_inv_ic = 0.f;
    if (next) {
        g.emit_bin = (uint8_t *)next->bin_src; g.emit_a = next->a;
        g.e_wp = next->wp; g.e_hp = next->hp; g.e_lead = next->lead; g.e_icp = next->icp;
        g.e_inv_ic = next->inv_ic;
        g.n_inner = 1;
    }
    // instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N and M encoded
    // (M = 256 for a pair: 128 rows in each CTA)
    g.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.n_tile >> 3) << 17) |
              ((uint32_t)((pair ? 2 * BM : BM) >> 4) << 24);
    // matrix descriptor, upper half: stride between 8-row groups (8 * kchunk bytes, in 16-byte
    // units), descriptor version 1, swizzle mode
    const uint32_t sbo = (uint32_t)(8 * p.kchunk) >> 4;
    const uint32_t layout = p.kchunk == 128 ? 2u : p.kchunk == 64 ? 4u : 6u;
    g.desc_hi = sbo | (1u << 14) | (layout << 29);
    g.a_bytes = (uint32_t)(BM * p.kchunk);
    g.tx_bytes = g.a_bytes + (uint32_t)(b_rows * p.kchunk);  // per CTA
    g.stage_bytes = (g.tx_bytes + 1023u) & ~1023u;
    g.issuers = g.taps * g.chunks_per_tap < 2 ? 1 : 2;
    g.kk_last = (p.ic - (g.chunks_per_tap - 1) * p.kchunk + 31) / 32;
    // as many ring buffers as fit beside the control block
    const size_t room = 227 * 1024 - 1024 - kControlBytes;
    g.halo = 0; g.n_a_slots = 0; g.a_slot_bytes = 0; g.b_ring_off = 0; g.b_slot_bytes = 0;
    g.b_bytes = (uint32_t)(b_rows * p.kchunk);
    bool halo = pair && p.kchunk == 128 && p.kw >= 2 && p.kw <= 9 && g.issuers <= p.kw;
    if (halo) {
        // three halo tiles of 136 positions, the rest of the room for filter tiles
        g.halo = BM + 8;
        g.n_a_slots = 3;
        g.a_slot_bytes = (uint32_t)(g.halo * p.kchunk + 1023) & ~1023u;
        g.b_slot_bytes = (g.b_bytes + 1023u) & ~1023u;
        g.b_ring_off = (uint32_t)g.n_a_slots * g.a_slot_bytes;
        g.n_stages = (int)((room - g.b_ring_off) / g.b_slot_bytes);
        if (g.n_stages > kMaxStages) g.n_stages = kMaxStages;
        if (g.n_stages < 4) { g.halo = 0; halo = false; }
    }
    if (!halo) {
        g.n_stages = (int)(room / g.stage_bytes);
        if (g.n_stages > kMaxStages) g.n_stages = kMaxStages;
    }
    if (g.n_stages < 2) return cudaErrorNotSupported;
    CUtensorMap map_a, map_b;
    if (!encode_bytes_2d(&map_a, bin_src, (uint64_t)p.rows, (uint64_t)p.icp, (uint32_t)p.kchunk,
                         (uint32_t)(halo ? g.halo : BM)) ||
        !encode_bytes_2d(&map_b, bin_w, (uint64_t)p.kh * p.kw * p.ocp16, (uint64_t)p.icp,
                         (uint32_t)p.kchunk, (uint32_t)b_rows))
        return cudaErrorNotSupported;

    const int kk = p.kchunk / 32;
    void (*kernel)(CUtensorMap, CUtensorMap, TcArgs) =
        pair ? (kk == 4   ? conv_tcgen05_kernel<4, true>
                : kk == 2 ? conv_tcgen05_kernel<2, true>
                          : conv_tcgen05_kernel<1, true>)
             : (kk == 4   ? conv_tcgen05_kernel<4, false>
                : kk == 2 ? conv_tcgen05_kernel<2, false>
                          : conv_tcgen05_kernel<1, false>);
    size_t smem = 1024 + kControlBytes +
                  (halo ? (size_t)g.b_ring_off + (size_t)g.n_stages * g.b_slot_bytes
                        : (size_t)g.n_stages * g.stage_bytes);
    // At least 120 KB of shared memory so that one CTA owns the SM and all 512 TMEM columns.
    if (smem < 120 * 1024) smem = 120 * 1024;
    // per device and kernel, once: the opt-in to large dynamic shared memory, the SM count and
    // the number of CTA pairs that can be resident together
    static std::atomic<bool> opted_in[64][3][2];
    std::atomic<bool> &done = opted_in[d][kk == 4 ? 0 : kk == 2 ? 1 : 2][pair ? 1 : 0];
    if (!done.load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(
            kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        done.store(true, std::memory_order_release);
    }
    note_launch();
    if (pair) {
        int pairs = pair_count[d].load(std::memory_order_relaxed);
        if (!pairs) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * (sms / 2));
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = 227 * 1024 - 1024;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&pairs, kernel, &cfg) != cudaSuccess || pairs <= 0) {
                (void)cudaGetLastError();
                pairs = sms / 2;
            }
            pair_count[d].store(pairs, std::memory_order_relaxed);
        }
        const int tiles = ((m_tiles + 1) / 2) * g.n_tiles;
        const int clusters = tiles < pairs ? tiles : pairs;
        return launch_overlapped(kernel, dim3(2 * clusters), dim3(kThreads), smem, s, 2, map_a, map_b, g);
    }
    const int tiles = g.n_inner ? g.m_tiles : g.m_tiles * g.n_tiles;
    const int grid = tiles < sms ? tiles : sms;
    return launch_overlapped(kernel, dim3(grid), dim3(kThreads), smem, s, 1, map_a, map_b, g);
}

}  // namespace xb200
