"""The allocation-free K entry point against the regular calculate_k executor.

xnor_nn_b200_calculate_k_noalloc exists for hosts that cannot allocate device memory at the
moment they need K (stream capture in progress, a server arena that owns the whole GPU, a plugin
sandbox). It keeps its mean-|x| scratch in an array built into the library, which every call on
the device shares and which keeps the previous call's values. So the check is made twice in a
row, the second time on a smaller layer with different data, to show that nothing left over from
the first call leaks into the second. Collected last on purpose: a failure here cannot mask
another test when the run stops at the first failure."""
import ctypes as C

import numpy as np
import pytest

import xnor_nn_b200 as xb
from xnor_nn_b200 import synth

pytestmark = pytest.mark.gpu


def _k_both_ways(torch, mb, oc, ic, ih, iw, kh, kw, ph, pw, seed, src_fmt=xb.NCHW):
    src = synth.normal(seed, mb * ic * ih * iw).reshape(mb, ic, ih, iw)
    if src_fmt == xb.NHWC:
        src = np.ascontiguousarray(src.transpose(0, 2, 3, 1))
    d_src = torch.from_numpy(src).cuda()
    conv = xb.Convolution(xb.ALGORITHM_BCAST, src_fmt, xb.OIHW, xb.NCHW, mb, oc, ic, ih, iw, kh,
                          kw, 1, 1, ph, pw)
    # existing entry point: the calculate_k executor, result read back from its slot
    assert conv.execute("calculate_k", src=d_src) == xb.SUCCESS
    conv.synchronize()
    want = conv.read(xb.SLOT_K, np.float32).copy()
    # new entry point: caller-owned device buffers, nothing allocated by the library
    d_k = torch.full((want.size,), float("nan"), device="cuda")
    st = xb.lib().xnor_nn_b200_calculate_k_noalloc(C.byref(conv.c), d_src.data_ptr(),
                                                   d_k.data_ptr(), None)
    assert st == xb.SUCCESS, xb.lib().xnor_nn_b200_noalloc_last_error()
    torch.cuda.synchronize()
    got = d_k.cpu().numpy()
    conv.close()
    return got, want


def test_noalloc_k_matches_executor_on_two_calls_in_a_row():
    torch = pytest.importorskip("torch")
    # 1st call: AlexNet conv4 geometry, 8 images; 2nd call: a smaller 5x5 layer, NHWC source
    got, want = _k_both_ways(torch, 8, 16, 384, 13, 13, 3, 3, 1, 1, seed=11)
    assert np.array_equal(got, want)   # same kernels, same order of additions: identical floats
    got, want = _k_both_ways(torch, 2, 8, 20, 9, 11, 5, 5, 2, 2, seed=12, src_fmt=xb.NHWC)
    assert np.array_equal(got, want)


def test_noalloc_refuses_what_it_cannot_serve():
    torch = pytest.importorskip("torch")
    L = xb.lib()
    limit = L.xnor_nn_b200_noalloc_max_pixels()
    # more pixels than the built-in scratch holds: refused before anything is launched
    big = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, 4, 8, 1, 1024,
                         limit // 4096 + 1, 3, 3, 1, 1, 1, 1)
    buf = torch.zeros(16, device="cuda")
    st = L.xnor_nn_b200_calculate_k_noalloc(C.byref(big.c), buf.data_ptr(), buf.data_ptr(), None)
    assert st == xb.ERROR_INVALID_INPUT
    assert b"exceeds" in L.xnor_nn_b200_noalloc_last_error()
    big.close()
    # host memory is not staged
    small = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, 1, 8, 4, 5, 5, 3, 3, 1,
                           1, 1, 1)
    host = np.zeros(4 * 25, np.float32)
    st = L.xnor_nn_b200_calculate_k_noalloc(C.byref(small.c), host.ctypes.data, buf.data_ptr(),
                                            None)
    assert st == xb.ERROR_INVALID_INPUT
    small.close()
