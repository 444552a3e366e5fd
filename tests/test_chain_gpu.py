"""Chained layers: consecutive binary convolutions whose intermediate results never exist as
floats (xnor_nn_b200_forward_chain). The reference for a chain is the layers run one after the
other: oracle convolution, then the oracle again on its float result.

What must hold: the packed signs handed to the next layer are exact, so that layer's integer sums
are bit-exact; its mean-|x| map is summed in a different (fixed) order than upstream's sequential
loop, so A, K and the final floats agree to rounding and are reproducible run to run."""
import numpy as np
import pytest

import xnor_nn_b200 as xb
from oracle.pyoracle import Shape
from xnor_nn_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4      # the float tolerance of the parity contract
A_REL_TOL = 1e-5    # mean-|x| map: a reordered sum of a few hundred non-negative terms


def _layer(mb, ic, oc, ih, iw, k, pad, kernel=None):
    return dict(mb=mb, ic=ic, oc=oc, ih=ih, iw=iw, kh=k, kw=k, ph=pad, pw=pad, kernel=kernel)


def _build(layers, seed):
    convs, weights, shapes = [], [], []
    for i, d in enumerate(layers):
        w = synth.normal(seed + 17 * i, d["oc"] * d["ic"] * d["kh"] * d["kw"], 0.05)
        convs.append(xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, d["mb"], d["oc"],
                                    d["ic"], d["ih"], d["iw"], d["kh"], d["kw"], 1, 1, d["ph"],
                                    d["pw"], w, kernel=d["kernel"]))
        weights.append(w)
        shapes.append(Shape.make(d["mb"], d["oc"], d["ic"], d["ih"], d["iw"], d["kh"], d["kw"], 1, 1,
                                 d["ph"], d["pw"], 0, 0, 0))
    return convs, weights, shapes


def _out_hw(d):
    return d["ih"] + 2 * d["pw"] - d["kh"] + 1, d["iw"] + 2 * d["pw"] - d["kw"] + 1


CHAINS = {
    "two_small": [_layer(2, 40, 48, 9, 11, 3, 1), _layer(2, 48, 24, 9, 11, 3, 1)],
    "shrinking_then_padded": [_layer(3, 20, 72, 12, 12, 3, 0), _layer(3, 72, 33, 10, 10, 5, 2)],
    "two_filter_tiles_feed_the_next": [_layer(1, 16, 260, 6, 6, 3, 1), _layer(1, 260, 40, 6, 6, 3, 1)],
    "alexnet_conv3_4_5": [_layer(2, 256, 384, 13, 13, 3, 1), _layer(2, 384, 256, 13, 13, 3, 1),
                          _layer(2, 256, 256, 13, 13, 3, 1)],
    "one_by_one_middle": [_layer(2, 64, 130, 7, 7, 3, 1), _layer(2, 130, 96, 7, 7, 1, 0),
                          _layer(2, 96, 16, 7, 7, 3, 1)],
}


@pytest.mark.parametrize("name", list(CHAINS))
def test_chain_equals_layer_by_layer(oracle, name):
    layers = CHAINS[name]
    convs, weights, shapes = _build(layers, 1000 + len(name))
    d0 = layers[0]
    src = synth.normal(77 + len(name), d0["mb"] * d0["ic"] * d0["ih"] * d0["iw"])
    if name == "two_small":
        src[: d0["ic"] * d0["ih"] * d0["iw"]] = 0.0   # an all-zero image: K = 0, results are +-0
    x = src
    want = None
    for shape, w in zip(shapes, weights):
        want = oracle.convolution(shape, x, w)
        x = want["dst"]
    got = np.full(want["dst"].size, np.nan, np.float32)
    xb.forward_chain(convs, src, got)
    # the last layer's packed input came from the previous layer's epilogue: exact signs
    assert np.array_equal(convs[-1].forward_sums(), want["sums"])
    a = convs[-1].read(xb.SLOT_A, np.float32)
    assert np.all(np.abs(a - want["a"]) <= A_REL_TOL * np.abs(want["a"]))
    err = np.abs(got - want["dst"])
    assert np.all(err <= REL_TOL * np.abs(want["dst"]))
    assert np.array_equal(got == 0, want["dst"] == 0)
    # reproducible: a second pass gives the same bytes
    again = np.empty_like(got)
    xb.forward_chain(convs, src, again)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
    # and the chain leaves every layer usable on its own afterwards
    alone = np.empty(int(np.prod(convs[0].out_shape)), np.float32)
    convs[0].forward(src, alone)
    first = oracle.convolution(shapes[0], src, weights[0])["dst"]
    assert np.all(np.abs(alone - first) <= REL_TOL * np.abs(first))
    for cv in convs:
        cv.close()


def test_chain_with_device_tensors_and_one_layer():
    torch = pytest.importorskip("torch")
    layers = CHAINS["two_small"]
    convs, weights, shapes = _build(layers, 5)
    d0 = layers[0]
    src = synth.normal(3, d0["mb"] * d0["ic"] * d0["ih"] * d0["iw"])
    host = np.empty(int(np.prod(convs[-1].out_shape)), np.float32)
    xb.forward_chain(convs, src, host)
    dsrc = torch.from_numpy(src).cuda()
    ddst = torch.empty(host.size, device="cuda")
    xb.forward_chain(convs, dsrc, ddst)
    convs[0].synchronize()
    assert np.array_equal(ddst.cpu().numpy(), host)
    # a chain of one is the ordinary fused call
    one = np.empty(int(np.prod(convs[0].out_shape)), np.float32)
    ref = np.empty_like(one)
    xb.forward_chain(convs[:1], src, one)
    convs[0].forward(src, ref)
    assert np.array_equal(one, ref)
    for cv in convs:
        cv.close()


def test_chain_refuses_layers_that_do_not_fit():
    a = _layer(2, 8, 16, 6, 6, 3, 1)
    convs, _, _ = _build([a, _layer(2, 24, 8, 6, 6, 3, 1)], 1)        # ic != previous oc
    src = np.ones(2 * 8 * 36, np.float32)
    dst = np.empty(2 * 8 * 36, np.float32)
    with pytest.raises(xb.XnorNNError) as e:
        xb.forward_chain(convs, src, dst)
    assert e.value.status == xb.ERROR_INVALID_INPUT
    convs, _, _ = _build([a, _layer(2, 16, 8, 5, 6, 3, 1)], 1)        # ih != previous oh
    with pytest.raises(xb.XnorNNError) as e:
        xb.forward_chain(convs, src, dst)
    assert e.value.status == xb.ERROR_INVALID_INPUT
    convs, _, _ = _build([a, _layer(2, 16, 8, 6, 6, 3, 1, kernel=xb.KERNEL_POPC)], 1)
    with pytest.raises(xb.XnorNNError) as e:
        xb.forward_chain(convs, src, dst)
    assert e.value.status == xb.UNIMPLEMENTED


def test_full_size_chain_conv3_conv4_matches_the_layers_run_separately():
    """AlexNet conv3 -> conv4 at the benchmark's minibatch, device resident: integer sums of the
    second layer bit-exact, floats to rounding, against the same library run layer by layer."""
    torch = pytest.importorskip("torch")
    mb = 256
    layers = [_layer(mb, 256, 384, 13, 13, 3, 1), _layer(mb, 384, 256, 13, 13, 3, 1)]
    convs, _, _ = _build(layers, 42)
    src = torch.from_numpy(synth.normal(9, mb * 256 * 169)).cuda()
    mid = torch.empty(mb * 384 * 169, device="cuda")
    want = torch.empty(mb * 256 * 169, device="cuda")
    convs[0].forward(src, mid)
    convs[1].forward(mid, want)
    convs[1].synchronize()
    sums_want = convs[1].forward_sums()
    got = torch.empty_like(want)
    xb.forward_chain(convs, src, got)
    convs[0].synchronize()
    assert np.array_equal(convs[1].forward_sums(), sums_want)
    w, g = want.cpu().numpy(), got.cpu().numpy()
    assert np.all(np.abs(g - w) <= 1e-5 * np.abs(w))
    for cv in convs:
        cv.close()
