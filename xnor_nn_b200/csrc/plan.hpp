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
    kPopc = 0,          // bits, LOP3 + POPC on the integer pipe; any stride, padding and format
    kTcgen05 = 2,       // +-1 int8, tcgen05.mma kind::i8 into tensor memory; stride 1
    kTcgen05Rows = 3,   // request only: the same family, forced onto its image-row kernel
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

    // ---- tiling of the image-row kernel (kTcgen05, conv_tcgen05_img.cu) ---------------------
    // That kernel puts 128 filters on the UMMA M side and, on the N side, `img_rows` whole output
    // rows of one image (img_rows * ow <= 256 positions, rounded up to 16 for the instruction).
    // Tiles are dealt round-robin to one CTA per SM; the tiles of a last, partly filled round are
    // cut in two row halves so that they spread over twice as many SMs.
    bool img;            // the forward pass launches the image-row kernel (else the position-tile one)
    bool img_forced;     // asked for by name, or the position-tile kernel cannot serve the shape
    int img_rows;        // output rows per tile
    int img_n;           // UMMA N of a whole tile
    int img_row_blocks;  // tiles per image column = ceil(oh / img_rows)
    int img_m_blocks;    // ceil(oc / 128)
    int img_tiles;       // mb * img_row_blocks * img_m_blocks
    int img_whole;       // tiles [0, img_whole) run whole, the rest as two halves each
    int img_half_rows;   // rows of the first half (0: nothing is split)
    int img_n_half;      // UMMA N of a half tile
    int img_grid;        // CTAs launched
    int img_stages;      // operand pipeline depth
    int img_staging;     // result staging buffers shared by the four epilogue warps (1, 2 or 4)

    size_t bytes[xnor_nn_resource_number];
};

int div_up_i(int a, int b);

// Fills a Plan from the descriptor fields and the requested family (kAuto: pick by shape).
// Never fails: unknown formats are remembered and reported by the executors.
void make_plan(Plan *p, const xnor_nn_convolution_t *c, Family requested);

// (Re)derives the image-row tiling from the plan's geometry and minibatch; called by make_plan and
// for every minibatch slice of a plan. Leaves p->img false when the shape does not suit.
void plan_image_rows(Plan *p);
// Result staging of the image-row kernel: words per filter row when every filter's run is staged
// on its own (room for a shift of up to three words; an odd multiple of 4, so that the rows of 32
// filters spread over the shared-memory banks as well as a multiple of 4 can), and
// bytes of one staging buffer (32 rows, or a dense 32 x OH*OW block for whole-image tiles).
int img_staging_row_words(const Plan &p);
size_t img_staging_bytes(const Plan &p);

const char *family_name(Family f);

}  // namespace xb200
