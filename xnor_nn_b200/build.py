"""Builds libxnor_nn.so (the drop-in shared library) in-tree with nvcc for sm_100a.

    python -m xnor_nn_b200.build [--force] [--verbose]

The library is the product: C++ host code and CUDA kernels behind the C interface declared in
include/xnor_nn.h and include/xnor_nn_b200.h. It links the CUDA runtime statically and reaches
the one driver call it needs (tensor-map encoding) through cudaGetDriverEntryPoint, so it has no
link-time dependency on libcuda and compiles on a machine without a GPU.
"""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libxnor_nn.so")
PROBE_SRC = os.path.join(CSRC, "probe", "pipe_probe.cu")
PROBE = os.path.join(PKG, "pipe_probe")
ISSUE_SRC = os.path.join(CSRC, "probe", "issue_probe.cu")
ISSUE = os.path.join(PKG, "issue_probe")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
          "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-ccbin", "/usr/bin/g++"]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile what changed and relink. Returns the path of the shared library."""
    os.makedirs(OBJ, exist_ok=True)
    headers = (glob.glob(os.path.join(CSRC, "*.h*")) + glob.glob(os.path.join(CSRC, "*.cuh")) +
               glob.glob(os.path.join(ROOT, "include", "*.h")) + [os.path.abspath(__file__)])
    objs, procs = [], []
    for src in _sources():
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) + \
                  ["-x", "cu", "-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("== %s\n%s\n" % (os.path.basename(src), out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or force or _stale(LIB, objs):
        cmd = [NVCC] + ARCH + ["-shared", "-cudart", "static", "-ccbin", "/usr/bin/g++",
                               "-o", LIB] + objs
        subprocess.check_call(cmd)
    # The pipe-rate probe is a stand-alone program (measured ceilings for the benchmark).
    if force or _stale(PROBE, [PROBE_SRC, os.path.abspath(__file__)]):
        subprocess.check_call([NVCC] + ARCH + ["-O3", "-std=c++17", "-lineinfo", "-ccbin",
                                               "/usr/bin/g++", "-o", PROBE, PROBE_SRC])
    # ... and so is the probe of instruction issue costs (profiles/ quotes its output).
    if force or _stale(ISSUE, [ISSUE_SRC, os.path.join(CSRC, "tc_ptx.cuh"), os.path.abspath(__file__)]):
        subprocess.check_call([NVCC] + ARCH + ["-O3", "-std=c++17", "-lineinfo", "-ccbin",
                                               "/usr/bin/g++", "-o", ISSUE, ISSUE_SRC])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
