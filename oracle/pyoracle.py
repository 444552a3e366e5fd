"""ctypes bindings for the two CPU checkers. TEST INFRASTRUCTURE ONLY.

`Oracle` wraps liboracle.so (the plain-C restatement in xnor_oracle.c); `UpstreamRef` wraps
_ref/libxnor_nn_ref.so (the unmodified upstream library, built by `make -C oracle ref` where the
upstream sources are present). Only the test-suite, the smoke check and the benchmark's CPU
baseline import this module; the product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libxnor_nn_ref.so")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def build(ref=True):
    """Compile liboracle.so, and the upstream library when its sources are on this machine."""
    subprocess.check_call(["make", "-s", "-C", HERE, "oracle"] + (["ref"] if ref else []))


class Shape(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("mb", "ic", "ih", "iw", "oc", "oh", "ow", "kh", "kw", "sh", "sw", "ph", "pw",
                 "src_nhwc", "w_hwio", "dst_nhwc")]

    @classmethod
    def make(cls, mb, oc, ic, ih, iw, kh, kw, sh=1, sw=1, ph=0, pw=0,
             src_nhwc=0, w_hwio=0, dst_nhwc=0):
        s = cls(mb=mb, ic=ic, ih=ih, iw=iw, oc=oc, kh=kh, kw=kw, sh=sh, sw=sw, ph=ph, pw=pw,
                src_nhwc=src_nhwc, w_hwio=w_hwio, dst_nhwc=dst_nhwc)
        # same arithmetic as upstream init (height uses pw)
        s.oh = (ih + 2 * pw - kh) // sh + 1
        s.ow = (iw + 2 * pw - kw) // sw + 1
        return s


class Oracle:
    def __init__(self, path=ORACLE_SO):
        if not os.path.exists(path):
            build(ref=False)
        L = self.lib = C.CDLL(path)
        sp = C.POINTER(Shape)
        L.oracle_abic.restype = C.c_int
        L.oracle_ico.restype = C.c_int
        L.oracle_binarize_data_bytes.argtypes = [sp, _f32p, C.c_int, _u8p]
        L.oracle_binarize_weights_bytes.argtypes = [sp, _f32p, C.c_int, C.c_int, _u8p]
        L.oracle_alpha.argtypes = [sp, _f32p, _f32p]
        L.oracle_operations_count.argtypes = [sp, _i32p]
        L.oracle_calculate_a_k.argtypes = [sp, _f32p, _f32p, _f32p]
        L.oracle_sums_from_bytes.argtypes = [sp, _u8p, _u8p, _i32p, C.c_int, C.c_int, _i32p]
        L.oracle_sums_from_floats.argtypes = [sp, _f32p, _f32p, _i32p]
        L.oracle_scale_store.argtypes = [sp, _i32p, _f32p, _f32p, _f32p]
        for f in ("oracle_binarize_data_bytes", "oracle_binarize_weights_bytes", "oracle_alpha",
                  "oracle_operations_count", "oracle_calculate_a_k", "oracle_sums_from_bytes",
                  "oracle_sums_from_floats", "oracle_scale_store"):
            getattr(L, f).restype = None

    def abic(self, ic, bici):
        return self.lib.oracle_abic(ic, bici)

    def ico(self, ic, bici):
        return self.lib.oracle_ico(ic, bici)

    def data_bytes(self, s, src, bici):
        out = np.empty(s.mb * s.ih * s.iw * self.abic(s.ic, bici), np.uint8)
        self.lib.oracle_binarize_data_bytes(C.byref(s), src.ravel(), bici, out)
        return out

    def weight_bytes(self, s, w, bici, oci):
        n = -(-s.oc // oci) * s.kh * s.kw * self.ico(s.ic, bici) * oci * bici
        out = np.empty(n, np.uint8)
        self.lib.oracle_binarize_weights_bytes(C.byref(s), w.ravel(), bici, oci, out)
        return out

    def alpha(self, s, w):
        out = np.empty(s.oc, np.float32)
        self.lib.oracle_alpha(C.byref(s), w.ravel(), out)
        return out

    def op_count(self, s):
        out = np.empty(s.oh * s.ow, np.int32)
        self.lib.oracle_operations_count(C.byref(s), out)
        return out

    def a_k(self, s, src):
        a = np.empty(s.mb * s.ih * s.iw, np.float32)
        k = np.empty(s.mb * s.oh * s.ow, np.float32)
        self.lib.oracle_calculate_a_k(C.byref(s), src.ravel(), a, k)
        return a, k

    def sums_from_bytes(self, s, bsrc, bw, bici, oci):
        out = np.empty(s.mb * s.oc * s.oh * s.ow, np.int32)
        self.lib.oracle_sums_from_bytes(C.byref(s), bsrc, bw, self.op_count(s), bici, oci, out)
        return out

    def sums(self, s, src, w):
        out = np.empty(s.mb * s.oc * s.oh * s.ow, np.int32)
        self.lib.oracle_sums_from_floats(C.byref(s), src.ravel(), w.ravel(), out)
        return out

    def scale_store(self, s, sums, alpha, k):
        out = np.empty(s.mb * s.oc * s.oh * s.ow, np.float32)
        self.lib.oracle_scale_store(C.byref(s), sums, alpha, k, out)
        return out

    def convolution(self, s, src, w):
        """Returns dict(dst, sums, alpha, a, k); dst is flat in the layout s.dst_nhwc names."""
        sums = self.sums(s, src, w)
        alpha = self.alpha(s, w)
        a, k = self.a_k(s, src)
        return dict(dst=self.scale_store(s, sums, alpha, k), sums=sums, alpha=alpha, a=a, k=k)


# ---- the unmodified upstream library -----------------------------------------------------------

_N_RES = 9
_EXEC = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_void_p))


class UpstreamConv(C.Structure):
    """xnor_nn_convolution_t as laid out by upstream include/xnor_nn_types.h:61-83."""
    _fields_ = ([("algorithm", C.c_int), ("mb", C.c_int), ("ic", C.c_int), ("ih", C.c_int),
                 ("iw", C.c_int), ("oc", C.c_int), ("oh", C.c_int), ("ow", C.c_int),
                 ("sh", C.c_int), ("sw", C.c_int), ("kh", C.c_int), ("kw", C.c_int),
                 ("ph", C.c_int), ("pw", C.c_int), ("src_format", C.c_int),
                 ("weights_format", C.c_int), ("dst_format", C.c_int),
                 ("resource_size", C.c_size_t * _N_RES),
                 ("binarize_weights", _EXEC), ("binarize_data", _EXEC), ("calculate_k", _EXEC),
                 ("forward", _EXEC), ("state", C.c_void_p)])


class UpstreamRef:
    """Drives the unmodified upstream library through its public C interface.

    XNOR_NN_ISA=2 is exported before the library initialises: on AVX-512 hosts upstream's
    default dispatch is wrong by its own tests (see oracle/Makefile).
    """
    ALG_REFERENCE, ALG_BCAST = 0, 1
    SLOT_SRC, SLOT_W, SLOT_DST, SLOT_ALPHA, SLOT_BSRC, SLOT_BW, SLOT_A, SLOT_K, SLOT_OPC = range(9)

    def __init__(self, path=REF_SO):
        os.environ.setdefault("XNOR_NN_ISA", "2")
        self.lib = C.CDLL(path)
        self.lib.xnor_nn_init_convolution.argtypes = [C.POINTER(UpstreamConv)] + [C.c_int] * 15
        self.lib.xnor_nn_allocate_resources.argtypes = [C.POINTER(UpstreamConv),
                                                       C.POINTER(C.c_void_p)]
        self.lib.xnor_nn_free_resources.argtypes = [C.POINTER(C.c_void_p)]
        self.lib.xnor_nn_destroy_convolution.argtypes = [C.POINTER(UpstreamConv)]

    @staticmethod
    def available(path=REF_SO):
        return os.path.exists(path)

    def run(self, s, src, w, algorithm=1, unit_scales=False, want_packed=False, timer=None):
        """One forward pass on the CPU. With unit_scales the alpha and K buffers are overwritten
        with 1.0f before `forward`, so dst carries the integer sums exactly. Returns a dict with
        dst (flat), alpha, a, k and, on request, the packed byte buffers."""
        c = UpstreamConv()
        st = self.lib.xnor_nn_init_convolution(
            C.byref(c), algorithm, 1 if s.src_nhwc else 0, 3 if s.w_hwio else 2,
            1 if s.dst_nhwc else 0, s.mb, s.oc, s.ic, s.ih, s.iw, s.kh, s.kw, s.sh, s.sw,
            s.ph, s.pw)
        assert st == 0
        res = (C.c_void_p * _N_RES)()
        assert self.lib.xnor_nn_allocate_resources(C.byref(c), res) == 0
        src = np.ascontiguousarray(src, np.float32).ravel()
        w = np.ascontiguousarray(w, np.float32).ravel()
        dst = np.empty(c.mb * c.oc * c.oh * c.ow, np.float32)
        res[0] = src.ctypes.data
        res[1] = w.ctypes.data
        res[2] = dst.ctypes.data
        out = {}
        try:
            import time
            t = {}
            for name in ("binarize_weights", "binarize_data", "calculate_k"):
                t0 = time.perf_counter()
                assert getattr(c, name)(C.addressof(c), res) == 0, name
                t[name] = time.perf_counter() - t0

            def view(slot, dtype, n):
                return np.ctypeslib.as_array(C.cast(res[slot], C.POINTER(dtype)), (n,)).copy()

            out["alpha"] = view(self.SLOT_ALPHA, C.c_float, c.oc)
            out["a"] = view(self.SLOT_A, C.c_float, c.mb * c.ih * c.iw)
            out["k"] = view(self.SLOT_K, C.c_float, c.mb * c.oh * c.ow)
            if want_packed:
                out["bin_src"] = view(self.SLOT_BSRC, C.c_uint8, c.resource_size[self.SLOT_BSRC])
                out["bin_weights"] = view(self.SLOT_BW, C.c_uint8,
                                          c.resource_size[self.SLOT_BW])
                out["sizes"] = list(c.resource_size)
            if unit_scales:
                nk = c.mb * c.oh * c.ow
                ones = np.ones(max(c.oc, nk), np.float32)
                C.memmove(res[self.SLOT_ALPHA], ones.ctypes.data, 4 * c.oc)
                C.memmove(res[self.SLOT_K], ones.ctypes.data, 4 * nk)
            t0 = time.perf_counter()
            assert c.forward(C.addressof(c), res) == 0
            t["forward"] = time.perf_counter() - t0
            if timer is not None:
                timer.update(t)
            out["dst"] = dst
            out["oh"], out["ow"] = c.oh, c.ow
        finally:
            self.lib.xnor_nn_free_resources(res)
            self.lib.xnor_nn_destroy_convolution(C.byref(c))
        return out
