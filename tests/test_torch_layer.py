"""The PyTorch layer over the library: upstream's Caffe layer
(external/caffe/src/caffe/layers/xnor_nn_conv_layer.cpp) restated for device tensors.

Forward must equal the oracle's convolution of the same input and weights; backward must be the
float convolution backward upstream describes (weights gradient from the real input, input
gradient through sign(w) * mean(w)); changed weights must be re-binarised."""
import numpy as np
import pytest

import cases
import xnor_nn_b200 as xb

torch = pytest.importorskip("torch")
from xnor_nn_b200.torch_layer import XnorConv2d  # noqa: E402

REL_TOL = 1e-4


def test_layer_is_lazy_and_refuses_host_tensors():
    layer = XnorConv2d(6, 16, 3, padding=1)
    assert layer.weight.shape == (16, 6, 3, 3) and not layer._convs
    with pytest.raises(ValueError, match="no CPU path"):
        layer(torch.zeros(1, 6, 5, 5))


def _case(name):
    return [c for c in cases.ALL_CASES if c[0] == name][0]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["alexnet_conv4", "cifar_32to64", "stride2", "ph0_pw1"])
def test_forward_matches_the_oracle(oracle, name):
    case = _case(name)
    d = case[1]
    src, w = cases.make_inputs(case)
    want = oracle.convolution(cases.oracle_shape(case), src, w)["dst"]
    layer = XnorConv2d(d["ic"], d["oc"], (d["kh"], d["kw"]), (d["sh"], d["sw"]),
                       (d["ph"], d["pw"])).cuda()
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w.reshape(layer.weight.shape)))
        x = torch.from_numpy(src.reshape(d["mb"], d["ic"], d["ih"], d["iw"])).cuda()
        y = layer(x)
        torch.cuda.synchronize()
    got = y.cpu().numpy().ravel()
    assert got.shape == want.shape
    assert np.all(np.abs(got - want) <= REL_TOL * np.abs(want))


@pytest.mark.gpu
def test_changed_weights_are_rebinarised_and_bias_is_added(oracle):
    case = _case("cifar_32to64")
    d = case[1]
    src, w = cases.make_inputs(case)
    layer = XnorConv2d(d["ic"], d["oc"], (d["kh"], d["kw"]), (d["sh"], d["sw"]),
                       (d["ph"], d["pw"]), bias=True).cuda()
    x = torch.from_numpy(src.reshape(d["mb"], d["ic"], d["ih"], d["iw"])).cuda()
    with torch.no_grad():
        layer.bias.copy_(torch.arange(d["oc"], dtype=torch.float32))
        for flip in (1.0, -1.0):      # second pass: every weight changes sign, in place
            layer.weight.copy_(torch.from_numpy(flip * w.reshape(layer.weight.shape)))
            y = layer(x).cpu().numpy()
            want = oracle.convolution(cases.oracle_shape(case), src, (flip * w).astype(np.float32))
            want = want["dst"].reshape(y.shape) + np.arange(d["oc"], dtype=np.float32).reshape(1, -1, 1, 1)
            assert np.all(np.abs(y - want) <= REL_TOL * np.abs(want) + 1e-6)


@pytest.mark.gpu
def test_backward_is_the_float_convolution_upstream_describes():
    torch.manual_seed(5)
    layer = XnorConv2d(12, 32, 3, padding=1, bias=True).cuda()
    x = torch.randn(4, 12, 9, 9, device="cuda", requires_grad=True)
    y = layer(x)
    gy = torch.randn_like(y)
    y.backward(gy)
    w = layer.weight.detach()
    # input gradient: through sign(w) * mean(w) (src/binarize_weights_float.cpp:3-25)
    bw = torch.where(w >= 0, 1.0, -1.0) * w.double().mean().float()
    want_gx = torch.nn.grad.conv2d_input(x.shape, bw, gy, padding=1)
    want_gw = torch.nn.grad.conv2d_weight(x.detach(), w.shape, gy, padding=1)
    assert torch.allclose(x.grad, want_gx, rtol=1e-3, atol=1e-6 * float(gy.abs().max()))
    assert torch.allclose(layer.weight.grad, want_gw, rtol=1e-4, atol=1e-4)
    assert torch.allclose(layer.bias.grad, gy.sum(dim=(0, 2, 3)), rtol=1e-5, atol=1e-4)
    assert layer._weights_changed  # the next forward pass binarises the weights again


@pytest.mark.gpu
def test_binarize_weights_float_on_the_device_matches_the_host_helper():
    """Signs exact; the mean within rounding of the index-order sum (the tolerance is relative
    to mean|w|, because the signed mean itself is a cancelling sum), and reproducible."""
    rng = np.random.default_rng(11)
    for oc, ic, k in ((256, 384, 3), (7, 3, 1), (512, 512, 3)):
        w = (rng.standard_normal(oc * ic * k * k) * 0.05 + 0.001).astype(np.float32)
        conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, 1, oc, ic, 8, 8,
                              k, k, 1, 1, 0, 0)
        host = np.empty_like(w)
        conv.binarize_weights_float(w, host)
        dw = torch.from_numpy(w).cuda()
        out = torch.empty_like(dw)
        conv.binarize_weights_float(dw, out)                       # upstream symbol, device pointers
        again = torch.empty_like(dw)
        conv.binarize_weights_float(dw, again, stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.array_equal(got, again.cpu().numpy())
        assert np.array_equal(np.signbit(got), np.signbit(host))
        assert abs(abs(got[0]) - abs(host[0])) <= 1e-5 * np.abs(w).mean()
        assert np.all(np.abs(got) == np.abs(got[0]))
        conv.binarize_weights_float(dw, dw, stream=torch.cuda.current_stream().cuda_stream)  # in place
        torch.cuda.synchronize()
        assert np.array_equal(dw.cpu().numpy(), got)
        conv.close()
