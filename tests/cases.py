"""Shapes shared by the CPU and GPU tests, and the builders of their inputs.

A case is (name, dict(mb, oc, ic, ih, iw, kh, kw, sh, sw, ph, pw), fill, formats) where fill is
"affine" (the two fills of upstream's differential test), "normal" or "uniform" (seeded), and
formats = (src_nhwc, w_hwio, dst_nhwc). Inputs are always generated as NCHW / OIHW and permuted
to the requested format, so a case means the same tensor in every layout.
"""
import hashlib
import zlib

import numpy as np

from xnor_nn_b200 import synth


def _c(name, mb, oc, ic, ih, iw, kh, kw, sh=1, sw=1, ph=0, pw=0, fill="normal", fmt=(0, 0, 0)):
    return (name, dict(mb=mb, oc=oc, ic=ic, ih=ih, iw=iw, kh=kh, kw=kw, sh=sh, sw=sw, ph=ph,
                       pw=pw), fill, fmt)


# Channel tails of upstream's differential suite
# (test/gtest/test_convolution_compare_with_reference.cpp:96-121): IC = 3..16, 24, 25, 26.
TAIL_CASES = [_c("tail_ic%d" % ic, 3, 8, ic, 13, 13, 3, 3, ph=1, pw=1, fill="affine")
              for ic in list(range(3, 17)) + [24]] + [
    _c("tail_ic%d_5x5" % ic, 1, 32, ic, 27, 27, 5, 5, ph=2, pw=2, fill="affine")
    for ic in (24, 25, 26)]

SHAPE_CASES = [
    # "task" layers (same file, lines 82-87), incl. the non-square 60x61 image
    _c("task_1to32", 1, 16, 1, 60, 61, 3, 3, fill="affine"),
    _c("task_32to32", 2, 32, 32, 20, 20, 3, 3, fill="affine"),
    # AlexNet conv1: stride 4, 11x11 (lines 148-149), fewer filters to keep the fixture small
    _c("alexnet_conv1_s4", 1, 16, 3, 227, 227, 11, 11, sh=4, sw=4),
    _c("alexnet_conv2", 1, 32, 96, 27, 27, 5, 5, ph=2, pw=2),
    _c("alexnet_conv3", 1, 384, 256, 13, 13, 3, 3, ph=1, pw=1),
    _c("alexnet_conv4", 1, 256, 384, 13, 13, 3, 3, ph=1, pw=1),
    _c("alexnet_conv4_affine", 2, 64, 384, 13, 13, 3, 3, ph=1, pw=1, fill="affine"),
    _c("vgg_512", 1, 48, 512, 28, 28, 3, 3, ph=1, pw=1, fill="uniform"),
    # cifar / mnist layers (lines 196-217)
    _c("cifar_3to32", 1, 32, 3, 32, 32, 5, 5, ph=2, pw=2),
    _c("cifar_32to64", 1, 64, 32, 32, 32, 5, 5, ph=2, pw=2),
    _c("mnist_1to24", 2, 24, 1, 28, 28, 5, 5),
    _c("mnist_24to48", 2, 48, 24, 8, 8, 5, 5),
    # odd sizes: filters not a multiple of 8, a stride-2 layer, unequal paddings (upstream
    # derives the output height from pw, src/common_convolution.cpp:16)
    _c("odd_oc13_ic70", 2, 13, 70, 9, 11, 3, 3, ph=1, pw=1),
    _c("stride2", 2, 24, 40, 17, 15, 3, 3, sh=2, sw=2, ph=1, pw=1),
    _c("ph0_pw1", 1, 16, 20, 9, 9, 3, 3, ph=0, pw=1),
    _c("one_by_one", 2, 40, 130, 7, 7, 1, 1),
    _c("single_pixel_out", 1, 8, 33, 3, 3, 3, 3),
    _c("oc260_two_filter_tiles", 1, 260, 16, 6, 6, 3, 3, ph=1, pw=1),
    # padding as large as the filter or larger: outputs that see no input pixel at all are 0
    _c("pad_ge_filter_1x1", 2, 24, 20, 5, 6, 1, 1, ph=1, pw=1),
    _c("pad_ge_filter_3x3", 1, 16, 40, 4, 5, 3, 3, ph=3, pw=3),
    # many small tiles: more work units than SMs, so CTAs of the persistent tensor-core kernels
    # run several tiles back to back (both accumulators, wrapped pipeline phases), and a thin
    # last round, which the image-row kernel cuts into half tiles
    _c("split_tail_152_tiles", 38, 512, 8, 4, 4, 3, 3, ph=1, pw=1),
    _c("three_rounds_450_tiles", 150, 384, 8, 2, 2, 3, 3, ph=1, pw=1),
    # more position tiles than SMs: the position-tile kernel runs them on CTA pairs. 151 tiles (an
    # odd count: the last pair's second CTA owns no position at all, and 76 pair tiles are two
    # rounds for two of the 74 pairs); two filter tiles of 192 with an odd number of position
    # tiles; an NHWC result
    _c("pairs_151_tiles", 2140, 32, 40, 2, 2, 3, 3, ph=1, pw=1),
    _c("pairs_two_filter_tiles_of_192", 1060, 384, 8, 2, 2, 3, 3, ph=1, pw=1),
    # the same with 128-byte channel chunks, where one position tile with a halo serves all taps of
    # a filter row: two chunks with a tail of 72 channels, 3x3; one chunk, 5x5
    _c("pairs_halo_ic200", 2140, 32, 200, 2, 2, 3, 3, ph=1, pw=1),
    _c("pairs_halo_5x5", 1205, 32, 128, 2, 2, 5, 5, ph=2, pw=2),
    # a filter tile that does not split into two UMMA-sized halves (48 filters): as many tiles, but
    # on single CTAs, each with two tiles or one
    _c("many_tiles_single_ctas", 2140, 48, 40, 2, 2, 3, 3, ph=1, pw=1),
    # many blocks of the activation packer on sources of one channel chunk (96 channels: chunks of
    # 96; 100: a chunk of 128 with a channel tail)
    _c("packer_many_blocks_ic96", 250, 16, 96, 13, 13, 3, 3, ph=1, pw=1),
    _c("packer_many_blocks_ic100", 250, 16, 100, 13, 13, 3, 3, ph=1, pw=1),
]

# Tensor formats other than NCHW/OIHW/NCHW
# (test/gtest/test_convolution_reference_forward.cpp:76-100 exercises all four combinations).
FORMAT_CASES = [
    _c("fmt_nchw_oihw_nhwc", 2, 24, 37, 6, 7, 3, 3, ph=1, pw=1, fmt=(0, 0, 1)),
    _c("fmt_nhwc_hwio_nchw", 2, 24, 37, 6, 7, 3, 3, ph=1, pw=1, fmt=(1, 1, 0)),
    _c("fmt_nhwc_hwio_nhwc", 2, 24, 37, 6, 7, 3, 3, ph=1, pw=1, fmt=(1, 1, 1)),
    # NHWC results whose rows are not whole 32-byte sectors (20 filters) or not even 16-byte
    # aligned (13 filters): the narrower store paths of the tensor-core epilogue
    _c("fmt_nhwc_dst_oc20", 2, 20, 37, 6, 7, 3, 3, ph=1, pw=1, fmt=(0, 0, 1)),
    _c("fmt_nhwc_dst_oc13", 2, 13, 37, 6, 7, 3, 3, ph=1, pw=1, fmt=(0, 0, 1)),
    _c("fmt_nhwc_dst_pairs", 2140, 32, 8, 2, 2, 3, 3, ph=1, pw=1, fmt=(0, 0, 1)),
]

ALL_CASES = TAIL_CASES + SHAPE_CASES + FORMAT_CASES


def case_seed(name):
    return zlib.crc32(name.encode()) & 0x7FFFFFFF


def make_inputs(case):
    """(src, weights) float32 arrays in the case's formats."""
    name, d, fill, fmt = case
    n_src = d["mb"] * d["ic"] * d["ih"] * d["iw"]
    n_w = d["oc"] * d["ic"] * d["kh"] * d["kw"]
    if fill == "affine":
        src = synth.upstream_fill_src(d["mb"], d["ic"], d["ih"], d["iw"])
        w = synth.upstream_fill_weights(d["oc"], d["ic"], d["kh"], d["kw"])
    else:
        seed = case_seed(name)
        gen = synth.normal if fill == "normal" else synth.uniform
        src = gen(seed, n_src).reshape(d["mb"], d["ic"], d["ih"], d["iw"])
        w = synth.normal(seed + 1, n_w, 0.05).reshape(d["oc"], d["ic"], d["kh"], d["kw"])
    if fmt[0]:
        src = np.ascontiguousarray(src.transpose(0, 2, 3, 1))
    if fmt[1]:
        w = np.ascontiguousarray(w.transpose(2, 3, 1, 0))
    return np.ascontiguousarray(src, np.float32), np.ascontiguousarray(w, np.float32)


def oracle_shape(case):
    from oracle.pyoracle import Shape
    _, d, _, fmt = case
    return Shape.make(d["mb"], d["oc"], d["ic"], d["ih"], d["iw"], d["kh"], d["kw"], d["sh"],
                      d["sw"], d["ph"], d["pw"], fmt[0], fmt[1], fmt[2])


def golden_sums_match(golden, name, sums):
    """Integer sums against the fixture, which holds them in full or, for the largest cases, as
    the SHA-256 of their int16 form."""
    if name + "/sums" in golden.files:
        return np.array_equal(sums, golden[name + "/sums"].astype(np.int32))
    s16 = np.asarray(sums).astype(np.int16)
    if not np.array_equal(s16.astype(np.int32), np.asarray(sums).astype(np.int32)):
        return False
    digest = np.frombuffer(hashlib.sha256(s16.tobytes()).digest(), np.uint8)
    return np.array_equal(digest, golden[name + "/sums_sha256"])
