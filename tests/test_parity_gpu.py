"""Parity of the CUDA path with the CPU oracle and with the committed upstream fixture.

Everything goes through the C interface (ctypes on libxnor_nn.so). Integer sums, alpha, A and K
are compared bit for bit; the scaled floats within 1e-4 relative (and, since A, K and alpha are
accumulated in upstream's order, they are in fact expected to be identical)."""
import ctypes as C

import numpy as np
import pytest

import cases
import xnor_nn_b200 as xb
from xnor_nn_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4  # the float tolerance of the parity contract
KERNELS = [xb.KERNEL_POPC, xb.KERNEL_TCGEN05_I8, xb.KERNEL_TCGEN05_I8_ROWS]


def _conv(case, kernel, weights):
    _, d, _, fmt = case
    return xb.Convolution(xb.ALGORITHM_BCAST, xb.NHWC if fmt[0] else xb.NCHW,
                          xb.HWIO if fmt[1] else xb.OIHW, xb.NHWC if fmt[2] else xb.NCHW,
                          d["mb"], d["oc"], d["ic"], d["ih"], d["iw"], d["kh"], d["kw"],
                          d["sh"], d["sw"], d["ph"], d["pw"], weights, kernel=kernel)


def _assert_close(got, want):
    err = np.abs(got - want)
    assert np.all(err <= REL_TOL * np.abs(want)), float((err / np.maximum(np.abs(want), 1e-30)).max())


@pytest.mark.parametrize("kernel", KERNELS, ids=[xb.KERNEL_NAMES[k] for k in KERNELS])
@pytest.mark.parametrize("case", cases.ALL_CASES, ids=[c[0] for c in cases.ALL_CASES])
def test_against_oracle_and_fixture(oracle, golden, case, kernel):
    name = case[0]
    src, w = cases.make_inputs(case)
    want = oracle.convolution(cases.oracle_shape(case), src, w)
    conv = _conv(case, kernel, w)
    dst = np.full(want["dst"].size, np.nan, np.float32)
    conv.forward(src, dst)
    sums = conv.forward_sums()
    # integers: bit-exact against the oracle and against upstream's own output
    assert np.array_equal(sums, want["sums"])
    assert cases.golden_sums_match(golden, name, sums)
    # scale factors: bit-exact
    assert np.array_equal(conv.read(xb.SLOT_ALPHA, np.float32), golden[name + "/alpha"])
    assert np.array_equal(conv.read(xb.SLOT_A, np.float32), golden[name + "/a"])
    assert np.array_equal(conv.read(xb.SLOT_K, np.float32), golden[name + "/k"])
    # floats: inside the contract's tolerance, and exactly zero where S is zero
    _assert_close(dst, want["dst"])
    assert np.array_equal(dst == 0, want["dst"] == 0)
    conv.close()


@pytest.mark.parametrize("kernel", KERNELS, ids=[xb.KERNEL_NAMES[k] for k in KERNELS])
def test_stepwise_executors_match_fused_call(oracle, kernel):
    """The literal upstream call sequence (three executors through the function pointers, host
    buffers) and the one-upload entry point give the same bytes; each executor can be repeated
    (upstream's perf harness calls them 4 to 128 times in a row,
    test/perf/test_simple_net.cpp:130-144)."""
    case = [c for c in cases.ALL_CASES if c[0] == "alexnet_conv2"][0]
    src, w = cases.make_inputs(case)
    conv = _conv(case, kernel, w)
    n = int(np.prod(conv.out_shape))
    a = np.empty(n, np.float32)
    b = np.empty(n, np.float32)
    conv.forward(src, a)
    conv.forward_stepwise(src, b)
    assert np.array_equal(a, b)
    for name in ("binarize_data", "binarize_data", "calculate_k", "calculate_k", "forward",
                 "forward"):
        assert conv.execute(name, src=src, dst=b) == xb.SUCCESS
    assert np.array_equal(a, b)
    conv.close()


@pytest.mark.parametrize("kernel", KERNELS, ids=[xb.KERNEL_NAMES[k] for k in KERNELS])
def test_device_pointers_skip_staging(oracle, kernel):
    """Tensors already on the device are used in place, on the caller's stream."""
    torch = pytest.importorskip("torch")
    case = [c for c in cases.ALL_CASES if c[0] == "alexnet_conv4"][0]
    src, w = cases.make_inputs(case)
    want = oracle.convolution(cases.oracle_shape(case), src, w)
    conv = _conv(case, kernel, torch.from_numpy(w).cuda())
    conv.set_stream(torch.cuda.current_stream().cuda_stream)
    d_src = torch.from_numpy(src).cuda()
    d_dst = torch.zeros(want["dst"].size, device="cuda")
    conv.forward(d_src, d_dst)
    d_sums = torch.zeros(want["sums"].size, dtype=torch.int32, device="cuda")
    conv.forward_sums(d_sums)
    torch.cuda.synchronize()
    assert np.array_equal(d_sums.cpu().numpy(), want["sums"])
    _assert_close(d_dst.cpu().numpy(), want["dst"])
    conv.close()


def test_host_pipeline_with_uneven_slices(oracle):
    """Host buffers of 8 MB or more go through the sliced upload/compute/download pipeline;
    41 images (10.6 MB) split into two unequal slices."""
    mb = 41
    L = synth.layer_shape("A", mb=mb)._replace(oc=32)
    src, w = synth.make_inputs("A", mb=mb)
    w = np.ascontiguousarray(w[:32])
    from oracle.pyoracle import Shape
    want = oracle.convolution(
        Shape.make(L.mb, L.oc, L.ic, L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw), src, w)
    for kernel in KERNELS:
        conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, L.mb, L.oc, L.ic,
                              L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w, kernel=kernel)
        dst = np.full(want["dst"].size, np.nan, np.float32)
        conv.forward(src, dst)
        assert np.array_equal(dst, want["dst"])
        assert np.array_equal(conv.read(xb.SLOT_K, np.float32), want["k"])
        conv.close()


def test_three_call_sequence_uploads_once(oracle):
    """Upstream's literal sequence with host buffers: binarize_data leaves the mean-|x| map of
    what it staged, the calculate_k that follows only box-filters it, and a calculate_k on its
    own (or on another tensor) still computes everything itself."""
    case = [c for c in cases.ALL_CASES if c[0] == "alexnet_conv4_affine"][0]
    src, w = cases.make_inputs(case)
    want = oracle.convolution(cases.oracle_shape(case), src, w)
    for kernel in KERNELS:
        conv = _conv(case, kernel, w)
        dst = np.full(want["dst"].size, np.nan, np.float32)
        conv.forward_stepwise(src, dst)
        assert np.array_equal(dst, want["dst"])
        assert np.array_equal(conv.read(xb.SLOT_A, np.float32), want["a"])
        # calculate_k alone, on a different tensor at a different address
        other = np.ascontiguousarray(src[::-1])
        assert conv.execute("calculate_k", src=other) == xb.SUCCESS
        want_other = oracle.convolution(cases.oracle_shape(case), other, w)
        assert np.array_equal(conv.read(xb.SLOT_K, np.float32), want_other["k"])
        # binarize_data then calculate_k on ANOTHER pointer: no shortcut
        assert conv.execute("binarize_data", src=src) == xb.SUCCESS
        assert conv.execute("calculate_k", src=other) == xb.SUCCESS
        assert np.array_equal(conv.read(xb.SLOT_A, np.float32), want_other["a"])
        conv.close()


def test_two_threads_share_one_descriptor(oracle):
    """One descriptor, one resource array per thread (each owns a stream and its staging
    buffers), as upstream allows: its executors only read the descriptor."""
    import threading
    case = [c for c in cases.ALL_CASES if c[0] == "alexnet_conv2"][0]
    src, w = cases.make_inputs(case)
    want = oracle.convolution(cases.oracle_shape(case), src, w)["dst"]
    first = _conv(case, None, w)
    results, errors = {}, []

    def work(tag):
        try:
            res = (C.c_void_p * xb.N_SLOTS)()
            L = xb.lib()
            assert L.xnor_nn_allocate_resources(C.byref(first.c), res) == xb.SUCCESS
            res[xb.SLOT_USER_WEIGHTS] = w.ctypes.data
            assert first.c.binarize_weights(C.addressof(first.c), res) == xb.SUCCESS
            out = np.empty(want.size, np.float32)
            for _ in range(5):
                res[xb.SLOT_USER_SRC] = src.ctypes.data
                res[xb.SLOT_USER_DST] = out.ctypes.data
                assert L.xnor_nn_b200_forward(C.byref(first.c), res) == xb.SUCCESS
            L.xnor_nn_free_resources(res)
            results[tag] = out
        except Exception as e:  # surfaced in the main thread
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for out in results.values():
        assert np.array_equal(out, want)
    first.close()


def test_more_filters_than_the_staged_alpha_table(oracle):
    """2100 filters: nine filter tiles, and alpha is read from global memory instead of the
    2048-entry shared-memory copy the tensor-core epilogue normally uses."""
    from oracle.pyoracle import Shape
    mb, oc, ic, ih, iw = 2, 2100, 16, 6, 6
    src = synth.normal(101, mb * ic * ih * iw).reshape(mb, ic, ih, iw)
    w = synth.normal(102, oc * ic * 9, 0.05).reshape(oc, ic, 3, 3)
    want = oracle.convolution(Shape.make(mb, oc, ic, ih, iw, 3, 3, 1, 1, 1, 1), src, w)
    conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, mb, oc, ic, ih, iw, 3, 3,
                          1, 1, 1, 1, w, kernel=xb.KERNEL_TCGEN05_I8)
    dst = np.empty(want["dst"].size, np.float32)
    conv.forward(src, dst)
    assert np.array_equal(conv.forward_sums(), want["sums"])
    assert np.array_equal(dst, want["dst"])
    conv.close()


def test_change_weights(oracle):
    case = [c for c in cases.ALL_CASES if c[0] == "mnist_24to48"][0]
    src, w = cases.make_inputs(case)
    conv = _conv(case, None, w)
    w2 = np.ascontiguousarray(-w[::-1])
    conv.change_weights(w2)
    dst = np.empty(int(np.prod(conv.out_shape)), np.float32)
    conv.forward(src, dst)
    _assert_close(dst, oracle.convolution(cases.oracle_shape(case), src, w2)["dst"])
    conv.close()


def test_reference_and_bcast_requests_agree():
    """Both algorithm requests are served by the same kernels, as the two upstream algorithms
    agree with each other."""
    case = [c for c in cases.ALL_CASES if c[0] == "task_32to32"][0]
    _, d, _, _ = case
    src, w = cases.make_inputs(case)
    outs = []
    for alg in (xb.ALGORITHM_REFERENCE, xb.ALGORITHM_BCAST):
        conv = xb.Convolution(alg, xb.NCHW, xb.OIHW, xb.NCHW, d["mb"], d["oc"], d["ic"], d["ih"],
                              d["iw"], d["kh"], d["kw"], d["sh"], d["sw"], d["ph"], d["pw"], w)
        dst = np.empty(int(np.prod(conv.out_shape)), np.float32)
        conv.forward(src, dst)
        outs.append(dst)
        conv.close()
    assert np.array_equal(outs[0], outs[1])


def test_unknown_format_is_unimplemented():
    """A format outside nchw/nhwc/oihw/hwio is refused by every executor with `unimplemented`
    (upstream src/bcast_binarize_data.cpp:36-38)."""
    conv = xb.Convolution(xb.ALGORITHM_BCAST, 7, xb.OIHW, xb.NCHW, 1, 8, 8, 5, 5, 3, 3, 1, 1, 1, 1)
    buf = np.zeros(8 * 8 * 5 * 5, np.float32)
    for name in ("binarize_weights", "binarize_data", "calculate_k", "forward"):
        assert conv.execute(name, src=buf, dst=buf, weights=buf) == xb.UNIMPLEMENTED
    conv.close()


def test_sign_of_negative_zero_follows_the_sign_bit():
    """-0.0 packs as negative and +0.0 as positive, the rule of upstream's packed path
    (src/bcast_binarize_data.cpp:61)."""
    src = np.array([0.0, -0.0, 1.0, -1.0], np.float32).reshape(1, 4, 1, 1)
    w = np.ones((1, 4, 1, 1), np.float32)
    conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, 1, 1, 4, 1, 1, 1, 1, 1, 1,
                          0, 0, w, kernel=xb.KERNEL_POPC)
    dst = np.empty(1, np.float32)
    conv.forward(src, dst)
    assert conv.forward_sums().tolist() == [0]  # +1 -1 +1 -1
    conv.close()


# ---- full-size layers: properties that need no oracle run --------------------------------------

FULL = ["B", "C", "D", "E"]


@pytest.mark.parametrize("cfg", FULL)
def test_full_size_properties(oracle, cfg):
    """At the benchmark sizes: (1) all kernels agree bit for bit on the integer sums, (2) the
    sums have the parity and range the operand count dictates, (3) negating the weights negates
    every sum, (4) for every kernel the first two and the last image are checked against the
    oracle: integer sums, mean-|x| and K maps bit for bit, scaled floats within 1e-4."""
    L = synth.CONFIGS[cfg]
    src, w = synth.make_inputs(cfg)
    ref_sums = None
    for kernel in KERNELS:
        conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, L.mb, L.oc, L.ic,
                              L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w, kernel=kernel)
        dst = np.full(int(np.prod(conv.out_shape)), np.nan, np.float32)
        conv.forward(src, dst)
        sums = conv.forward_sums()
        # floats, A and K at full size: the three oracle-checked images (1e-4 relative for the
        # results, bit for bit for the scale maps), and no result left unwritten anywhere
        assert not np.isnan(dst).any()
        from oracle.pyoracle import Shape
        a_map = conv.read(xb.SLOT_A, np.float32)
        k_map = conv.read(xb.SLOT_K, np.float32)
        for first in (0, L.mb - 1):
            n = 2 if first == 0 else 1
            s = Shape.make(n, L.oc, L.ic, L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw)
            want = oracle.convolution(s, src[first:first + n], w)
            per = L.oc * conv.c.oh * conv.c.ow
            _assert_close(dst[first * per:(first + n) * per], want["dst"])
            pa, pk = L.ih * L.iw, conv.c.oh * conv.c.ow
            assert np.array_equal(a_map[first * pa:(first + n) * pa], want["a"])
            assert np.array_equal(k_map[first * pk:(first + n) * pk], want["k"])
            assert np.array_equal(sums[first * per:(first + n) * per], want["sums"])
        if ref_sums is None:
            ref_sums = sums
            op_c = conv.read(xb.SLOT_OPERATIONS_COUNT, np.int32)
            s4 = sums.reshape(L.mb, L.oc, -1)
            assert np.all((s4 - op_c[None, None, :]) % 2 == 0)
            assert np.all(np.abs(s4) <= op_c[None, None, :])
            conv.change_weights(np.ascontiguousarray(-w))
            conv.forward(src, dst)
            assert np.array_equal(conv.forward_sums(), -sums)
        else:
            assert np.array_equal(sums, ref_sums), xb.KERNEL_NAMES[kernel]
        conv.close()
