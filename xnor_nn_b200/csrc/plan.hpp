// Host-side description of one binary convolution on the device: geometry, the kernel family
// chosen for it, and the layout of every internal buffer. One Plan hangs off
// xnor_nn_convolution_t::state (the role upstream's Implementation object plays,
// src/implementation.hpp:11-25); it is immutable after xnor_nn_init_convolution.
#pragma once

#include <cstddef>
#include <cstdint>

#include "xnor_nn.h"

namespace xb200 {

// Which convolution kernel consumes the packed operands. The packed layouts differ per family,
// so the choice is fixed at init and every executor of the descriptor follows it.
enum Family : int {
    kPopc = 0,     // bits, LOP3 + POPC on the integer pipe; any stride, padding and format
    kMmaB1 = 1,    // mma.sync m16n8k256 xor.popc: measured, ruled out, never selected
    kTcgen05 = 2,  // +-1 int8, tcgen05.mma kind::i8 into tensor memory; stride 1
    kAuto = -1,
};

struct Plan {
    // geometry (copied from the descriptor so kernels never chase the caller's struct)
    int mb, ic, ih, iw, oc, oh, ow, kh, kw, sh, sw, ph, pw;
    bool src_nhwc, w_hwio, dst_nhwc;
    bool formats_ok;  // false: an unknown tensor format was requested -> xnor_nn_unimplemented

    Family family;

    // scalars rounded on the host exactly as upstream computes them
    float inv_ic;   // 1.f / IC                     (src/bcast_calculate_k.cpp:42)
    float inv_khw;  // 1.f / KH / KW                (src/bcast_calculate_k.cpp:43)
    float inv_chw;  // 1.f / (IC*KH*KW)             (src/bcast_binarize_weights.cpp:95)

    // ---- bit layout (kPopc) -------------------------------------------------------------
    // activations: uint32 [mb][ih][iw][icw]; channel c is bit (31 - c%32) of word c/32; bits
    //              past the last channel are 0.
    // weights:     uint32 [kh][kw][icw][ocp]; same bit order, bits past the last channel 0,
    //              so absent channels xor to 0 on both sides.
    int icw;  // 32-bit words per pixel
    int ocp;  // output channels rounded up to the kernel's channel tile

    // ---- int8 layout (kTcgen05) ----------------------------------------------------------
    // Activations are +-1 bytes on a zero frame so that a filter tap is a constant row shift:
    // rows of (iw + pw) positions (the pw zeros after a row double as the left border of the
    // next one), (ih + ph) rows per image (same sharing between images), lead rows of zeros in
    // front. Position q of image n, row h, column w sits at row
    //   lead + (n*(ih+ph) + h)*(iw+pw) + w
    // of a [rows][icp] byte matrix, and tap (kh,kw) of the output at q reads row
    //   q + (kh-ph)*(iw+pw) + (kw-pw).
    int icp;        // channels rounded up to the K chunk (bytes per position)
    int kchunk;     // bytes of K per pipeline stage: 128, 64 or 32 (= the swizzle span)
    int wp, hp;     // iw + pw, ih + ph
    int lead;       // zero rows in front of the first image
    long rows;      // rows allocated (frame + tail slack so every tile load is in range)
    long q_total;   // positions the kernel computes (mb*hp*wp), a multiple of nothing
    int ocp16;      // output channels rounded up to 16 (UMMA N granularity)
    int n_tile;     // UMMA N per accumulator (<= 256, multiple of 16)

    size_t bytes[xnor_nn_resource_number];
};

int div_up_i(int a, int b);

// Fills a Plan from the descriptor fields and the requested family (kAuto: pick by shape).
// Never fails: unknown formats are remembered and reported by the executors.
void make_plan(Plan *p, const xnor_nn_convolution_t *c, Family requested);

const char *family_name(Family f);

}  // namespace xb200
