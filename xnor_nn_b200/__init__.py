"""xnor_nn for B200: Python binding of the drop-in C library (libxnor_nn.so).

The product is the shared library built from csrc/ (C++ host code and CUDA kernels for sm_100a
behind the upstream C interface). This module is the thin ctypes layer the tests and the
benchmark drive it through; `Convolution` mirrors upstream's C++ wrapper
(include/xnor_nn.hpp:11-68: constructor = init + allocate + binarize_weights, `forward`,
`change_weights`) with the same argument order and meaning.

There is no CPU fallback: loading fails if the library has not been built, and every call
returns a non-success status (raised here as XnorNNError) when no CUDA device is usable.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libxnor_nn.so")

# enumerators of include/xnor_nn.h
SUCCESS, ERROR_MEMORY, ERROR_INVALID_INPUT, UNIMPLEMENTED = range(4)
ALGORITHM_REFERENCE, ALGORITHM_BCAST, ALGORITHM_BEST = 0, 1, 1
NCHW, NHWC, OIHW, HWIO = 0, 1, 2, 3
(SLOT_USER_SRC, SLOT_USER_WEIGHTS, SLOT_USER_DST, SLOT_ALPHA, SLOT_BIN_SRC, SLOT_BIN_WEIGHTS,
 SLOT_A, SLOT_K, SLOT_OPERATIONS_COUNT) = range(9)
N_SLOTS = 9
KERNEL_AUTO, KERNEL_POPC, KERNEL_TCGEN05_I8, KERNEL_TCGEN05_I8_ROWS = -1, 0, 2, 3
KERNEL_NAMES = {KERNEL_POPC: "popc", KERNEL_TCGEN05_I8: "tcgen05_i8",
                KERNEL_TCGEN05_I8_ROWS: "tcgen05_i8_rows"}

_EXECUTOR = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_void_p))


class ConvolutionDesc(C.Structure):
    """xnor_nn_convolution_t, field for field (include/xnor_nn.h)."""
    _fields_ = [("algorithm", C.c_int), ("mb", C.c_int), ("ic", C.c_int), ("ih", C.c_int),
                ("iw", C.c_int), ("oc", C.c_int), ("oh", C.c_int), ("ow", C.c_int),
                ("sh", C.c_int), ("sw", C.c_int), ("kh", C.c_int), ("kw", C.c_int),
                ("ph", C.c_int), ("pw", C.c_int), ("src_format", C.c_int),
                ("weights_format", C.c_int), ("dst_format", C.c_int),
                ("resource_size", C.c_size_t * N_SLOTS),
                ("binarize_weights", _EXECUTOR), ("binarize_data", _EXECUTOR),
                ("calculate_k", _EXECUTOR), ("forward", _EXECUTOR), ("state", C.c_void_p)]


class XnorNNError(RuntimeError):
    def __init__(self, status, detail=""):
        self.status = status
        msg = status_message(status)
        super().__init__(msg + (": " + detail if detail else ""))


_lib = None


def lib():
    """The loaded shared library; raises if it was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -m xnor_nn_b200.build` "
                "(there is no CPU fallback)" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        dp = C.POINTER(ConvolutionDesc)
        rp = C.POINTER(C.c_void_p)
        L.xnor_nn_get_status_message.argtypes = [C.c_char_p, C.c_int]
        L.xnor_nn_get_status_message.restype = None
        L.xnor_nn_init_convolution.argtypes = [dp] + [C.c_int] * 15
        L.xnor_nn_b200_init_convolution.argtypes = [dp] + [C.c_int] * 16
        L.xnor_nn_allocate_resources.argtypes = [dp, rp]
        L.xnor_nn_free_resources.argtypes = [rp]
        L.xnor_nn_free_resources.restype = None
        L.xnor_nn_destroy_convolution.argtypes = [dp]
        L.xnor_nn_destroy_convolution.restype = None
        L.xnor_nn_binarize_weights_float.argtypes = [dp, C.c_void_p, C.c_void_p]
        L.xnor_nn_binarize_weights_float.restype = None
        L.xnor_nn_b200_binarize_weights_float.argtypes = [dp, C.c_void_p, C.c_void_p, C.c_void_p]
        L.xnor_nn_b200_kernel_of.argtypes = [dp]
        L.xnor_nn_b200_forward.argtypes = [dp, rp]
        L.xnor_nn_b200_binarize.argtypes = [dp, rp]
        L.xnor_nn_b200_forward_chain.argtypes = [C.c_int, C.POINTER(dp), C.POINTER(rp)]
        L.xnor_nn_b200_forward_sums.argtypes = [dp, rp, C.c_void_p]
        L.xnor_nn_b200_read_resource.argtypes = [dp, rp, C.c_int, C.c_void_p, C.c_size_t]
        L.xnor_nn_b200_set_stream.argtypes = [rp, C.c_void_p]
        L.xnor_nn_b200_get_stream.argtypes = [rp]
        L.xnor_nn_b200_get_stream.restype = C.c_void_p
        L.xnor_nn_b200_synchronize.argtypes = [rp]
        L.xnor_nn_b200_last_error.restype = C.c_char_p
        L.xnor_nn_b200_kernel_launches.restype = C.c_long
        L.xnor_nn_b200_forward_sharded.argtypes = [dp, rp, C.POINTER(C.c_int), C.c_int]
        L.xnor_nn_b200_selftest_lost_commit.argtypes = [dp, rp, C.c_uint]
        L.xnor_nn_b200_calculate_k_noalloc.argtypes = [dp, C.c_void_p, C.c_void_p, C.c_void_p]
        L.xnor_nn_b200_noalloc_max_pixels.restype = C.c_long
        L.xnor_nn_b200_noalloc_last_error.restype = C.c_char_p
        _lib = L
    return _lib


def status_message(status):
    buf = C.create_string_buffer(16)
    lib().xnor_nn_get_status_message(buf, status)
    return buf.value.decode()


def last_error():
    return lib().xnor_nn_b200_last_error().decode()


def kernel_launches():
    return lib().xnor_nn_b200_kernel_launches()


def _check(status):
    if status != SUCCESS:
        raise XnorNNError(status, last_error())


def _ptr(x):
    """Address of a numpy array (host), a torch tensor (host or device) or a raw integer."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if isinstance(x, np.ndarray):
        assert x.flags["C_CONTIGUOUS"]
        return x.ctypes.data
    if hasattr(x, "data_ptr"):
        assert x.is_contiguous()
        return x.data_ptr()
    raise TypeError(type(x))


class Convolution:
    """Mirror of upstream xnor_nn::Convolution (include/xnor_nn.hpp:11-68)."""

    def __init__(self, algorithm, src_fmt, weights_fmt, dst_fmt, MB, OC, IC, IH, IW, KH, KW,
                 SH, SW, PH, PW, weights=None, kernel=None):
        L = lib()
        self.c = ConvolutionDesc()
        self.res = (C.c_void_p * N_SLOTS)()
        self._keep = {}
        if kernel is None:
            _check(L.xnor_nn_init_convolution(C.byref(self.c), algorithm, src_fmt, weights_fmt,
                                              dst_fmt, MB, OC, IC, IH, IW, KH, KW, SH, SW, PH, PW))
        else:
            _check(L.xnor_nn_b200_init_convolution(C.byref(self.c), algorithm, src_fmt,
                                                   weights_fmt, dst_fmt, MB, OC, IC, IH, IW, KH,
                                                   KW, SH, SW, PH, PW, kernel))
        self._allocated = False
        _check(L.xnor_nn_allocate_resources(C.byref(self.c), self.res))
        self._allocated = True
        if weights is not None:
            self.change_weights(weights)

    # -- upstream surface ------------------------------------------------------------------
    def change_weights(self, weights):
        self._set(SLOT_USER_WEIGHTS, weights)
        _check(self.c.binarize_weights(C.addressof(self.c), self.res))

    def forward(self, src, dst):
        """binarize_data + calculate_k + forward, as upstream's wrapper does, issued through
        the one-upload entry point."""
        self._set(SLOT_USER_SRC, src)
        self._set(SLOT_USER_DST, dst)
        try:
            _check(lib().xnor_nn_b200_forward(C.byref(self.c), self.res))
        finally:
            self._clear_user_io()

    def forward_sharded(self, src, dst, devices, weights=None):
        """One pass of a host minibatch over several GPUs; `weights` (host array) is needed the
        first time a device list is used."""
        self._set(SLOT_USER_SRC, src)
        self._set(SLOT_USER_DST, dst)
        if weights is not None:
            self._set(SLOT_USER_WEIGHTS, weights)
        dev = (C.c_int * len(devices))(*devices)
        try:
            _check(lib().xnor_nn_b200_forward_sharded(C.byref(self.c), self.res, dev, len(devices)))
        finally:
            self._clear_user_io()
            self.res[SLOT_USER_WEIGHTS] = None
            self._keep.pop(SLOT_USER_WEIGHTS, None)

    def forward_stepwise(self, src, dst):
        """The literal upstream sequence: three executor calls through the function pointers."""
        self._set(SLOT_USER_SRC, src)
        self._set(SLOT_USER_DST, dst)
        try:
            for ex in (self.c.binarize_data, self.c.calculate_k, self.c.forward):
                _check(ex(C.addressof(self.c), self.res))
        finally:
            self._clear_user_io()

    def binarize_weights_float(self, src, dst, stream=None):
        """sign(src) * mean(src). Host arrays, or device tensors; with `stream` (device tensors
        only) the work is enqueued there and not waited for."""
        if stream is None:
            lib().xnor_nn_binarize_weights_float(C.byref(self.c), _ptr(src), _ptr(dst))
        else:
            _check(lib().xnor_nn_b200_binarize_weights_float(C.byref(self.c), _ptr(src),
                                                             _ptr(dst), stream))

    # -- single executors and extensions ---------------------------------------------------
    def execute(self, name, src=None, dst=None, weights=None):
        """Calls one executor (`binarize_weights`, `binarize_data`, `calculate_k`, `forward`)
        and returns its status code without raising."""
        if src is not None:
            self._set(SLOT_USER_SRC, src)
        if dst is not None:
            self._set(SLOT_USER_DST, dst)
        if weights is not None:
            self._set(SLOT_USER_WEIGHTS, weights)
        return getattr(self.c, name)(C.addressof(self.c), self.res)

    def forward_sums(self, out=None):
        n = self.c.mb * self.c.oc * self.c.oh * self.c.ow
        if out is None:
            out = np.empty(n, np.int32)
        _check(lib().xnor_nn_b200_forward_sums(C.byref(self.c), self.res, _ptr(out)))
        return out

    def read(self, slot, dtype):
        """Host copy of an internal slot, viewed as `dtype`."""
        nbytes = self.c.resource_size[slot]
        buf = np.empty(nbytes, np.uint8)
        _check(lib().xnor_nn_b200_read_resource(C.byref(self.c), self.res, slot,
                                                buf.ctypes.data, nbytes))
        return buf.view(dtype)

    def set_stream(self, stream_ptr):
        _check(lib().xnor_nn_b200_set_stream(self.res, stream_ptr))

    def synchronize(self):
        _check(lib().xnor_nn_b200_synchronize(self.res))

    @property
    def kernel(self):
        return lib().xnor_nn_b200_kernel_of(C.byref(self.c))

    @property
    def out_shape(self):
        c = self.c
        if c.dst_format == NHWC:
            return (c.mb, c.oh, c.ow, c.oc)
        return (c.mb, c.oc, c.oh, c.ow)

    def _set(self, slot, x):
        self._keep[slot] = x  # the library reads the pointer during the call: keep it alive
        self.res[slot] = _ptr(x)

    def _clear_user_io(self):
        # upstream's wrapper clears the two slots after every pass (include/xnor_nn.hpp:50-52);
        # the references go too, so a caller's tensors are not held until the next call
        for slot in (SLOT_USER_SRC, SLOT_USER_DST):
            self.res[slot] = None
            self._keep.pop(slot, None)

    def close(self):
        if getattr(self, "res", None) is not None and self._allocated:
            lib().xnor_nn_free_resources(self.res)
            self._allocated = False
        if getattr(self, "c", None) is not None and self.c.state:
            lib().xnor_nn_destroy_convolution(C.byref(self.c))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def forward_chain(convs, src, dst):
    """Runs `convs` (Convolution objects, in order) back to back without the float tensors
    between them: src -> convs[0] -> ... -> convs[-1] -> dst."""
    n = len(convs)
    cs = (C.POINTER(ConvolutionDesc) * n)(*[C.pointer(cv.c) for cv in convs])
    rs = (C.POINTER(C.c_void_p) * n)(*[C.cast(cv.res, C.POINTER(C.c_void_p)) for cv in convs])
    convs[0]._set(SLOT_USER_SRC, src)
    convs[-1]._set(SLOT_USER_DST, dst)
    try:
        _check(lib().xnor_nn_b200_forward_chain(n, cs, rs))
    finally:
        convs[0]._clear_user_io()
        convs[-1]._clear_user_io()
