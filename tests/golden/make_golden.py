"""Regenerates upstream_golden.npz, the fixture the parity tests are pinned to.

Run where the upstream sources are mounted (it needs oracle/_ref/libxnor_nn_ref.so, built by
`make -C oracle ref`):

    python tests/golden/make_golden.py

For every case of tests/cases.py the unmodified upstream library computes, through its public C
interface: dst (fp32; as a SHA-256 digest when large), alpha, A, K, and the integer sums S (as a
digest beyond 400 000 values; second run with alpha and K
overwritten by 1.0f, so that dst carries S exactly). Inputs are not stored: they are regenerated
from the case definition (affine fills, or the seeded generators of xnor_nn_b200/synth.py).

The three known-answer vectors of upstream's own test-suite are stored as literals:
  test/gtest/test_convolution_reference_forward.cpp:20-73   (convolution incl. border)
  test/gtest/test_data_bin_reference.cpp:20-53              (A and K incl. border)
  test/gtest/test_weights_bin_reference.cpp:19-50           (alpha)
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
from oracle.pyoracle import UpstreamRef  # noqa: E402

P, N = 1.0, -1.0
KAT = dict(
    kat_src_nchw=np.array([P, P, P, N, P, N, N, N, N,
                           N, N, N, N, N, N, P, P, P], np.float32),
    kat_src_nhwc=np.array([P, N, P, N, P, N, N, N, P, N, N, N, N, P, N, P, N, P], np.float32),
    kat_weights_oihw=np.array([P, P, P, N, N, P, P, N, N,
                               P, P, P, P, P, P, P, P, P,
                               N, N, N, N, N, N, N, N, N,
                               P, P, P, N, N, P, P, N, N], np.float32),
    kat_weights_hwio=np.array([P, N, P, P, P, N, P, P, P, N, P, P,
                               N, N, P, N, N, N, P, N, P, N, P, P,
                               P, N, P, P, N, N, P, N, N, N, P, N], np.float32),
    kat_dst_nchw_times9=np.array([-16, -48, -16, 24, 0, 0, 0, 0, 8,
                                  0, 0, 0, -24, -18, 0, 0, 0, -8], np.float32),
    kat_dst_nhwc_times9=np.array([-16, 0, -48, 0, -16, 0, 24, -24, 0, -18, 0, 0,
                                  0, 0, 0, 0, 8, -8], np.float32),
    kat_a=np.ones(9, np.float32),
    kat_k_times9=np.array([4, 6, 4, 6, 9, 6, 4, 6, 4], np.float32),
    kat_alpha=np.ones(2, np.float32),
)


def main():
    ref = UpstreamRef()
    out = dict(KAT)
    for case in cases.ALL_CASES:
        name, d, fill, fmt = case
        s = cases.oracle_shape(case)
        src, w = cases.make_inputs(case)
        # bcast serves NCHW/OIHW; upstream's tests only drive the other formats through the
        # reference algorithm, so do the same here
        alg = 1 if fmt == (0, 0, 0) else 0
        r = ref.run(s, src, w, algorithm=alg)
        ru = ref.run(s, src, w, algorithm=alg, unit_scales=True)
        sums = ru["dst"]
        if fmt[2]:  # stored NCHW-indexed whatever the result layout
            sums = np.ascontiguousarray(
                sums.reshape(d["mb"], r["oh"], r["ow"], d["oc"]).transpose(0, 3, 1, 2)).ravel()
        assert np.array_equal(sums, np.rint(sums)) and np.abs(sums).max() < 32768
        # dst in full only for small cases; otherwise its SHA-256 (the oracle must reproduce
        # upstream's floats bit for bit, so a digest pins it as well as the array would)
        if r["dst"].size <= 5000:
            out[name + "/dst"] = r["dst"]
        out[name + "/dst_sha256"] = np.frombuffer(
            hashlib.sha256(r["dst"].tobytes()).digest(), np.uint8)
        # the integer sums in full up to 400 000 of them, beyond that as the SHA-256 of their
        # int16 form (cases.golden_sums_match knows both)
        if sums.size <= 400000:
            out[name + "/sums"] = sums.astype(np.int16)
        else:
            out[name + "/sums_sha256"] = np.frombuffer(
                hashlib.sha256(sums.astype(np.int16).tobytes()).digest(), np.uint8)
        out[name + "/alpha"] = r["alpha"]
        out[name + "/a"] = r["a"]
        out[name + "/k"] = r["k"]
        print("%-24s outputs=%d  max|S|=%d" % (name, sums.size, np.abs(sums).max()))
    path = os.path.join(HERE, "upstream_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
