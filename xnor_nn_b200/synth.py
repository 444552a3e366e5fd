"""Seeded synthetic layers: the five benchmark shapes and the fills of the upstream test-suite.

Upstream measures on no dataset: its perf harness feeds a deterministic ramp
(test/perf/test_simple_net.cpp:91-93) and its differential test two affine fills
(test/gtest/test_convolution_compare_with_reference.cpp:9-27). The benchmark layers here are
named by shape and value distribution only, so everything is generated: a counter-based
SplitMix64 stream mapped to uniform or (Box-Muller) normal values. Exact zeros are never
produced, because the sign of -0.0 is the one input on which the two upstream algorithms
disagree (sign bit in src/bcast_binarize_data.cpp:61, `>= 0` in
src/reference_convolution.cpp:102).
"""
from collections import namedtuple

import numpy as np

Layer = namedtuple("Layer", "name mb oc ic ih iw kh kw sh sw ph pw src_dist src_scale w_scale")

# name: (batch, OC, IC, IH, IW, KH, KW, SH, SW, PH, PW, source distribution, scale, weight std)
CONFIGS = {
    "A": Layer("alexnet_conv4_mb1", 1, 256, 384, 13, 13, 3, 3, 1, 1, 1, 1, "normal", 1.0, 0.05),
    "B": Layer("alexnet_conv4_mb256", 256, 256, 384, 13, 13, 3, 3, 1, 1, 1, 1, "normal", 1.0, 0.05),
    "C": Layer("alexnet_conv3_mb256", 256, 384, 256, 13, 13, 3, 3, 1, 1, 1, 1, "normal", 1.0, 0.05),
    "D": Layer("alexnet_conv2_mb128", 128, 256, 96, 27, 27, 5, 5, 1, 1, 2, 2, "normal", 1.0, 0.05),
    "E": Layer("vgg_512_mb64", 64, 512, 512, 28, 28, 3, 3, 1, 1, 1, 1, "uniform", 1.0, 0.02),
}
SRC_SEED = 0x5EED0000
W_SEED = 0xBEEF0000


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15))
    z = x
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _uniform01(seed, n, stream):
    """n doubles in (0, 1), a pure function of (seed, stream, index)."""
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64)
        key = _splitmix64(np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream))
        bits = _splitmix64(idx ^ key)
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))


def normal(seed, n, std=1.0):
    u1 = _uniform01(seed, n, 1)
    u2 = _uniform01(seed, n, 2)
    v = (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std).astype(np.float32)
    return _no_zeros(v)


def uniform(seed, n, half_width=1.0):
    v = ((2.0 * _uniform01(seed, n, 3) - 1.0) * half_width).astype(np.float32)
    return _no_zeros(v)


def _no_zeros(v):
    v[v == 0] = np.float32(1e-30)
    assert not np.isnan(v).any()
    return v


def layer_shape(cfg, mb=None):
    L = CONFIGS[cfg] if isinstance(cfg, str) else cfg
    return L._replace(mb=mb) if mb is not None else L


def make_inputs(cfg, mb=None, first_image=0):
    """(src NCHW, weights OIHW) for a benchmark layer. Image i of the batch depends only on
    (config, i), so a minibatch slice [first_image, first_image+mb) equals the same slice of
    the full batch: this is what lets shards be generated independently."""
    L = layer_shape(cfg, mb)
    index = "ABCDE".index(cfg) if isinstance(cfg, str) else 0
    per = L.ic * L.ih * L.iw
    gen = normal if L.src_dist == "normal" else uniform
    src = np.empty((L.mb, L.ic, L.ih, L.iw), np.float32)
    for i in range(L.mb):
        src[i] = gen(SRC_SEED + index + 977 * (first_image + i + 1), per, L.src_scale).reshape(
            L.ic, L.ih, L.iw)
    w = normal(W_SEED + index, L.oc * L.ic * L.kh * L.kw, L.w_scale).reshape(
        L.oc, L.ic, L.kh, L.kw)
    return src, w


def upstream_fill_src(mb, ic, ih, iw):
    """0.33 + 0.0023*(19 - (iw+ih+ic+mb%37)), NCHW
    (test/gtest/test_convolution_compare_with_reference.cpp:9-17)."""
    m, c, h, w = np.ogrid[:mb, :ic, :ih, :iw]
    t = (19 - (w + h + c + m % 37)).astype(np.float32)
    return (np.float32(0.33) + np.float32(0.0023) * t).astype(np.float32)


def upstream_fill_weights(oc, ic, kh, kw):
    """0.18 + 0.017*(11 - (kw+kh+ic+oc%23)), OIHW (same file, lines 19-27)."""
    o, c, h, w = np.ogrid[:oc, :ic, :kh, :kw]
    t = (11 - (w + h + c + o % 23)).astype(np.float32)
    return (np.float32(0.18) + np.float32(0.017) * t).astype(np.float32)
