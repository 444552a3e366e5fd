"""xnor_nn_b200_forward_sharded: one call that spreads a host minibatch over a list of GPUs and
gathers the results in the caller's tensor. The two-device case needs two GPUs and is skipped on
a single-GPU machine; the argument checks and the one-device case run anywhere."""
import numpy as np
import pytest

import xnor_nn_b200 as xb
from xnor_nn_b200 import synth

pytestmark = pytest.mark.gpu


def _layer(mb):
    L = synth.layer_shape("A", mb=mb)._replace(oc=48)
    src, w = synth.make_inputs("A", mb=mb)
    return L, src, np.ascontiguousarray(w[:48])


def _want(oracle, L, src, w):
    from oracle.pyoracle import Shape
    return oracle.convolution(
        Shape.make(L.mb, L.oc, L.ic, L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw), src, w)


def _conv(L, w):
    return xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, L.mb, L.oc, L.ic, L.ih,
                          L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w)


def test_one_device_list_equals_the_plain_call(oracle):
    L, src, w = _layer(5)
    want = _want(oracle, L, src, w)
    conv = _conv(L, w)
    dst = np.full(want["dst"].size, np.nan, np.float32)
    conv.forward_sharded(src, dst, [0], weights=w)
    assert np.array_equal(dst, want["dst"])
    dst[:] = np.nan
    conv.forward_sharded(src, dst, [0])  # replicas are kept: no weights needed again
    assert np.array_equal(dst, want["dst"])
    conv.close()


def test_two_devices_slices_of_two_and_three_images(oracle):
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    L, src, w = _layer(5)
    want = _want(oracle, L, src, w)
    conv = _conv(L, w)
    h_src = torch.from_numpy(src).pin_memory()
    h_dst = torch.full((want["dst"].size,), float("nan")).pin_memory()
    conv.forward_sharded(h_src, h_dst, [0, 1], weights=w)
    assert np.array_equal(h_dst.numpy(), want["dst"])
    # another order of the same devices rebuilds the replicas
    h_dst.fill_(float("nan"))
    conv.forward_sharded(h_src, h_dst, [1, 0], weights=w)
    assert np.array_equal(h_dst.numpy(), want["dst"])
    conv.close()


def test_more_devices_than_images(oracle):
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    L, src, w = _layer(1)
    want = _want(oracle, L, src, w)
    conv = _conv(L, w)
    dst = np.full(want["dst"].size, np.nan, np.float32)
    conv.forward_sharded(src, dst, [0, 1], weights=w)  # device 0 gets nothing
    assert np.array_equal(dst, want["dst"])
    conv.close()


def test_argument_checks():
    torch = pytest.importorskip("torch")
    L, src, w = _layer(2)
    conv = _conv(L, w)
    dst = np.zeros(int(np.prod(conv.out_shape)), np.float32)
    with pytest.raises(xb.XnorNNError) as e:
        conv.forward_sharded(src, dst, [99], weights=w)  # no such device
    assert e.value.status == xb.ERROR_INVALID_INPUT
    with pytest.raises(xb.XnorNNError) as e:
        conv.forward_sharded(src, dst, [0, 0], weights=w)  # a device named twice
    assert e.value.status == xb.ERROR_INVALID_INPUT
    with pytest.raises(xb.XnorNNError) as e:
        conv.forward_sharded(src, dst, [0])  # first use of a device list without weights
    assert e.value.status == xb.ERROR_INVALID_INPUT
    with pytest.raises(xb.XnorNNError) as e:
        conv.forward_sharded(torch.from_numpy(src).cuda(), dst, [0], weights=w)
    assert e.value.status == xb.ERROR_INVALID_INPUT
    conv.close()
