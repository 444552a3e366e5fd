"""Host-side checks of the drop-in library that need no GPU: it loads, exports every symbol the
headers declare, lays the descriptor out like upstream, and reports errors by status code."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import xnor_nn_b200 as xb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    names = set()
    for h in ("xnor_nn.h", "xnor_nn_b200.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= {n for n in re.findall(r"\b(xnor_nn_[a-z0-9_]+)\s*\(", text)
                  if not n.endswith("_t")}
    return sorted(names)


def test_library_exports_every_declared_symbol():
    L = xb.lib()
    names = _declared_functions()
    assert "xnor_nn_init_convolution" in names and "xnor_nn_b200_forward" in names
    for n in names:
        assert hasattr(L, n), n


def test_status_messages():
    """Same strings as upstream src/status.cpp:3-15; the longest fits upstream's char[16]."""
    want = {0: "success", 1: "memory_error", 2: "bad_input", 3: "unimplemented"}
    for code, text in want.items():
        assert xb.status_message(code) == text


def test_descriptor_layout_matches_upstream_header():
    """Offsets a program compiled against upstream's header relies on (LP64)."""
    d = xb.ConvolutionDesc
    assert d.algorithm.offset == 0 and d.mb.offset == 4 and d.ic.offset == 8
    assert d.oc.offset == 20 and d.oh.offset == 24 and d.ow.offset == 28
    assert d.sh.offset == 32 and d.kh.offset == 40 and d.ph.offset == 48
    assert d.src_format.offset == 56 and d.dst_format.offset == 64
    assert d.resource_size.offset == 72
    assert d.binarize_weights.offset == 144 and d.binarize_data.offset == 152
    assert d.calculate_k.offset == 160 and d.forward.offset == 168 and d.state.offset == 176
    assert C.sizeof(d) == 184


def _init(kernel=None, **kw):
    p = dict(alg=xb.ALGORITHM_BCAST, sf=xb.NCHW, wf=xb.OIHW, df=xb.NCHW, mb=2, oc=16, ic=20,
             ih=9, iw=11, kh=3, kw=3, sh=1, sw=1, ph=1, pw=1)
    p.update(kw)
    c = xb.ConvolutionDesc()
    args = [p[k] for k in ("alg", "sf", "wf", "df", "mb", "oc", "ic", "ih", "iw", "kh", "kw",
                           "sh", "sw", "ph", "pw")]
    if kernel is None:
        st = xb.lib().xnor_nn_init_convolution(C.byref(c), *args)
    else:
        st = xb.lib().xnor_nn_b200_init_convolution(C.byref(c), *args, kernel)
    assert st == xb.SUCCESS
    return c


def test_init_fills_descriptor_like_upstream():
    c = _init(ih=227, iw=227, kh=11, kw=11, sh=4, sw=4, ph=0, pw=0, ic=3, oc=96)
    assert (c.oh, c.ow) == (55, 55)
    assert (c.mb, c.oc, c.ic) == (2, 96, 3)
    assert all(c.resource_size[i] > 0 for i in range(3, 9))
    assert c.resource_size[xb.SLOT_ALPHA] == 96 * 4
    assert c.resource_size[xb.SLOT_A] == 2 * 227 * 227 * 4
    assert c.resource_size[xb.SLOT_K] == 2 * 55 * 55 * 4
    assert c.state
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))
    assert not c.state


def test_output_height_uses_pw_like_upstream():
    """Upstream passes pw for both extents (src/common_convolution.cpp:16-17)."""
    c = _init(ih=9, iw=9, ph=0, pw=1)
    assert (c.oh, c.ow) == (9, 9)
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))


def test_kernel_family_selection():
    c = _init(kernel=xb.KERNEL_POPC)
    assert xb.lib().xnor_nn_b200_kernel_of(C.byref(c)) == xb.KERNEL_POPC
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))
    # the tensor-core families walk a unit-stride frame; a strided layer degrades to popc
    c = _init(kernel=xb.KERNEL_TCGEN05_I8, sh=2, sw=2)
    assert xb.lib().xnor_nn_b200_kernel_of(C.byref(c)) == xb.KERNEL_POPC
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))


def test_executors_reject_missing_slots():
    """NULL slots give bad_input before anything touches the device
    (upstream src/bcast_binarize_data.cpp:15-19 and siblings)."""
    c = _init()
    res = (C.c_void_p * xb.N_SLOTS)()
    for ex in (c.binarize_weights, c.binarize_data, c.calculate_k, c.forward):
        assert ex(C.addressof(c), res) == xb.ERROR_INVALID_INPUT
        assert ex(None, res) == xb.ERROR_INVALID_INPUT
    assert xb.lib().xnor_nn_b200_forward(C.byref(c), res) == xb.ERROR_INVALID_INPUT
    xb.lib().xnor_nn_free_resources(res)  # nothing allocated: must be harmless
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))


def test_unknown_slots_are_not_served():
    """Internal slots that this library did not create have no device context: bad_input."""
    c = _init()
    res = (C.c_void_p * xb.N_SLOTS)()
    junk = np.zeros(1 << 16, np.uint8)
    for i in range(xb.N_SLOTS):
        res[i] = junk.ctypes.data
    assert c.binarize_data(C.addressof(c), res) == xb.ERROR_INVALID_INPUT
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))


def test_binarize_weights_float_host_helper():
    """to = sign(from) * mean(from) (upstream src/binarize_weights_float.cpp:3-25)."""
    c = _init(oc=4, ic=3, kh=2, kw=2)
    w = np.linspace(-1.0, 2.0, 4 * 3 * 2 * 2).astype(np.float32)
    out = np.empty_like(w)
    xb.lib().xnor_nn_binarize_weights_float(C.byref(c), w.ctypes.data, out.ctypes.data)
    mean = np.float32(0)
    for v in w:
        mean = np.float32(mean + v)
    mean = np.float32(mean * np.float32(1.0 / w.size))
    np.testing.assert_array_equal(out, np.where(w >= 0, mean, -mean).astype(np.float32))
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="a GPU is present")
def test_no_cpu_fallback_without_a_device():
    """Without a CUDA device allocation fails with a status code and leaves every slot NULL;
    nothing computes on the host instead."""
    c = _init()
    res = (C.c_void_p * xb.N_SLOTS)()
    st = xb.lib().xnor_nn_allocate_resources(C.byref(c), res)
    assert st == xb.ERROR_MEMORY
    assert all(res[i] is None for i in range(3, 9))
    assert xb.last_error() != ""
    xb.lib().xnor_nn_destroy_convolution(C.byref(c))


def test_chain_and_device_helpers_reject_bad_arguments():
    """Argument checks of the entry points that have no upstream counterpart happen before any
    CUDA call, so they can be exercised without a device."""
    L = xb.lib()
    c = xb.ConvolutionDesc()
    assert L.xnor_nn_init_convolution(C.byref(c), 1, 0, 2, 0, 2, 16, 8, 6, 6, 3, 3, 1, 1, 1, 1) == 0
    res = (C.c_void_p * xb.N_SLOTS)()
    cs = (C.POINTER(xb.ConvolutionDesc) * 1)(C.pointer(c))
    rs = (C.POINTER(C.c_void_p) * 1)(C.cast(res, C.POINTER(C.c_void_p)))
    assert L.xnor_nn_b200_forward_chain(0, cs, rs) == xb.ERROR_INVALID_INPUT
    assert L.xnor_nn_b200_forward_chain(1, None, rs) == xb.ERROR_INVALID_INPUT
    assert L.xnor_nn_b200_forward_chain(1, cs, rs) == xb.ERROR_INVALID_INPUT   # nothing allocated
    w = np.ones(16 * 8 * 9, np.float32)
    # host memory where device memory is required
    assert L.xnor_nn_b200_binarize_weights_float(C.byref(c), w.ctypes.data, w.ctypes.data,
                                                 None) == xb.ERROR_INVALID_INPUT
    assert L.xnor_nn_b200_binarize_weights_float(C.byref(c), None, None, None) == xb.ERROR_INVALID_INPUT
    L.xnor_nn_destroy_convolution(C.byref(c))
