"""Pins the CPU oracle: against upstream's known-answer vectors, against the committed fixture
of upstream outputs, and (where the upstream build is present) against upstream run live,
including its packed byte layouts. All CPU."""
import hashlib

import numpy as np
import pytest

import cases
from oracle.pyoracle import Shape, UpstreamRef


def _sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), np.uint8)


# ---- upstream's own known-answer tests ---------------------------------------------------------

@pytest.mark.parametrize("src_nhwc,w_hwio,dst_nhwc", [(0, 0, 0), (0, 0, 1), (1, 1, 0), (1, 1, 1)])
def test_kat_convolution(oracle, golden, src_nhwc, w_hwio, dst_nhwc):
    """test/gtest/test_convolution_reference_forward.cpp: 1x2x3x3 -> 2 filters, 3x3, pad 1, in the
    four layout combinations. Upstream allows 1e-3 (test/gtest/common.hpp:146-161); 1e-5 here
    (K accumulates six to nine rounded 1/9 terms, so it is not the exact quotient)."""
    s = Shape.make(1, 2, 2, 3, 3, 3, 3, 1, 1, 1, 1, src_nhwc, w_hwio, dst_nhwc)
    src = golden["kat_src_nhwc" if src_nhwc else "kat_src_nchw"]
    w = golden["kat_weights_hwio" if w_hwio else "kat_weights_oihw"]
    r = oracle.convolution(s, src, w)
    want = golden["kat_dst_nhwc_times9" if dst_nhwc else "kat_dst_nchw_times9"] / np.float32(9)
    np.testing.assert_allclose(r["dst"], want, rtol=0, atol=1e-5)


@pytest.mark.parametrize("src_nhwc", [0, 1])
def test_kat_a_and_k(oracle, golden, src_nhwc):
    """test/gtest/test_data_bin_reference.cpp:43-53: A == 1, K = {4,6,4,6,9,6,4,6,4}/9, i.e. the
    box filter divides by KH*KW everywhere and adds nothing outside the image."""
    s = Shape.make(1, 2, 2, 3, 3, 3, 3, 1, 1, 1, 1, src_nhwc, 0, 0)
    a, k = oracle.a_k(s, golden["kat_src_nhwc" if src_nhwc else "kat_src_nchw"])
    np.testing.assert_allclose(a, golden["kat_a"], atol=1e-5)
    np.testing.assert_allclose(k, golden["kat_k_times9"] / 9.0, atol=1e-5)


@pytest.mark.parametrize("w_hwio", [0, 1])
def test_kat_alpha(oracle, golden, w_hwio):
    """test/gtest/test_weights_bin_reference.cpp:50: alpha == {1, 1}."""
    s = Shape.make(1, 2, 2, 3, 3, 3, 3, 1, 1, 1, 1, 0, w_hwio, 0)
    alpha = oracle.alpha(s, golden["kat_weights_hwio" if w_hwio else "kat_weights_oihw"])
    np.testing.assert_allclose(alpha, golden["kat_alpha"], atol=1e-5)


# ---- committed fixture of upstream outputs -----------------------------------------------------

@pytest.mark.parametrize("case", cases.ALL_CASES, ids=[c[0] for c in cases.ALL_CASES])
def test_oracle_matches_upstream_fixture(oracle, golden, case):
    """Bit-exact on everything: integer sums, alpha, A, K and the scaled floats."""
    name = case[0]
    s = cases.oracle_shape(case)
    src, w = cases.make_inputs(case)
    r = oracle.convolution(s, src, w)
    assert cases.golden_sums_match(golden, name, r["sums"])
    assert np.array_equal(r["alpha"], golden[name + "/alpha"])
    assert np.array_equal(r["a"], golden[name + "/a"])
    assert np.array_equal(r["k"], golden[name + "/k"])
    assert np.array_equal(_sha(r["dst"]), golden[name + "/dst_sha256"])
    if name + "/dst" in golden.files:
        assert np.array_equal(r["dst"], golden[name + "/dst"])


def test_operations_count(oracle):
    """op_c = IC * taps inside the image: 4/6/9 taps on a 3x3 image with a padded 3x3 filter."""
    s = Shape.make(1, 1, 5, 3, 3, 3, 3, 1, 1, 1, 1)
    assert oracle.op_count(s).tolist() == [20, 30, 20, 30, 45, 30, 20, 30, 20]


# ---- upstream run live -------------------------------------------------------------------------

live = pytest.mark.skipif(not UpstreamRef.available(),
                          reason="upstream build (oracle/_ref) not present on this machine")


@pytest.fixture(scope="module")
def upstream():
    return UpstreamRef()


LIVE = [c for c in cases.ALL_CASES if c[0] in (
    "tail_ic3", "tail_ic9", "tail_ic16", "tail_ic25_5x5", "task_1to32", "alexnet_conv1_s4",
    "alexnet_conv2", "alexnet_conv4", "mnist_24to48", "stride2", "ph0_pw1",
    "fmt_nhwc_hwio_nhwc")]


@live
@pytest.mark.parametrize("case", LIVE, ids=[c[0] for c in LIVE])
def test_oracle_matches_upstream_live(oracle, upstream, case):
    name, d, fill, fmt = case
    s = cases.oracle_shape(case)
    src, w = cases.make_inputs(case)
    alg = 1 if fmt == (0, 0, 0) else 0
    r = upstream.run(s, src, w, algorithm=alg, want_packed=True)
    sums = upstream.run(s, src, w, algorithm=alg, unit_scales=True)["dst"]
    if fmt[2]:
        sums = sums.reshape(d["mb"], s.oh, s.ow, d["oc"]).transpose(0, 3, 1, 2).ravel()
    mine = oracle.convolution(s, src, w)
    assert np.array_equal(mine["sums"].astype(np.float32), sums)
    for key in ("dst", "alpha", "a", "k"):
        assert np.array_equal(mine[key], r[key]), key
    # upstream's packed byte layouts (int16 word path, 16 filters per AVX vector)
    bici = 2 if d["ic"] * d["kh"] * d["kw"] < 32767 else 4
    oci = 32 // bici
    if alg == 1 and d["oc"] % oci == 0:
        bsrc = oracle.data_bytes(s, src, bici)
        bw = oracle.weight_bytes(s, w, bici, oci)
        assert np.array_equal(bsrc, r["bin_src"])
        assert np.array_equal(bw, r["bin_weights"][:bw.size])
        assert np.array_equal(oracle.sums_from_bytes(s, bsrc, bw, bici, oci), mine["sums"])


@live
def test_both_upstream_algorithms_agree(upstream):
    """The float-domain and the packed upstream algorithms give identical floats, which is what
    lets one GPU path stand in for both."""
    case = [c for c in cases.ALL_CASES if c[0] == "alexnet_conv2"][0]
    s = cases.oracle_shape(case)
    src, w = cases.make_inputs(case)
    a = upstream.run(s, src, w, algorithm=0)["dst"]
    b = upstream.run(s, src, w, algorithm=1)["dst"]
    assert np.array_equal(a, b)
