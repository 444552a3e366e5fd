"""Drop-in checks with compiled callers: upstream's own example programs and public-interface
test-suites, built unmodified against upstream's headers and linked with this library
(`make -C oracle dropin`, where the upstream sources are mounted), and this repository's C++
wrapper driven through upstream's known-answer case."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "oracle", "_ref", "dropin")


def _run(path, timeout=600):
    return subprocess.run([path], capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("name", ["simple_convolution_c", "simple_convolution_cpp"])
def test_upstream_examples_run_against_this_library(name):
    """example/simple_convolution.{c,cpp}: init, allocate, binarize_weights, three forward passes
    through the executor pointers, free; they print the final status."""
    exe = os.path.join(DROPIN, name)
    if not os.path.exists(exe):
        pytest.skip("drop-in binaries were not built on a machine with the upstream sources")
    r = _run(exe)
    assert r.returncode == 0, r.stdout + r.stderr
    if name.endswith("_c"):
        assert "success" in r.stdout


@pytest.mark.parametrize("name", ["gtest_reference_forward", "gtest_compare_with_reference"])
def test_upstream_gtest_suites_pass_against_this_library(name):
    """test_convolution_reference_forward.cpp (known answer incl. the border, four layouts) and
    test_convolution_compare_with_reference.cpp (94 shapes: channel tails 3..26, AlexNet conv1-5
    incl. the stride-4 layer, cifar, mnist) through upstream's own C++ wrapper, i.e. the literal
    three-executor call sequence with host buffers."""
    exe = os.path.join(DROPIN, name)
    if not os.path.exists(exe):
        pytest.skip("drop-in binaries were not built on a machine with the upstream sources")
    r = _run(exe, timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "PASSED" in r.stdout and "FAILED" not in r.stdout


def test_cpp_wrapper_known_answer(tmp_path):
    """include/xnor_nn.hpp on upstream's known-answer convolution, plus its exception path."""
    exe = str(tmp_path / "wrapper_kat")
    subprocess.check_call(["g++", "-std=c++14", "-Wall", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "wrapper_kat.cpp"), "-o", exe,
                           "-L", os.path.join(ROOT, "xnor_nn_b200"), "-lxnor_nn",
                           "-Wl,-rpath," + os.path.join(ROOT, "xnor_nn_b200")])
    r = _run(exe)
    assert r.returncode == 0, r.stdout + r.stderr
