"""Benchmark of the binary-convolution path on N B200s: AlexNet conv4, minibatch 256 (headline),
and the other four named layers beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config A..E|all] [--kernel auto|popc|tcgen05_i8|tcgen05_i8_rows]

A step is one forward pass of the layer (sign-pack + mean-|x| map, K box filter, XNOR/popcount
convolution with the alpha*K epilogue) over the whole minibatch; with N GPUs the minibatch is
split into N contiguous slices, one process per GPU, no collective on the data path (strong
scaling: the total batch stays fixed). Rank 0 prints one JSON line.

  value / ms_per_step  effective binary TOPS = 2*MB*OC*OH*OW*IC*KH*KW / time, tensors resident in
             HBM; the K timed steps are repeated as whole regions until 50 ms have been timed
             and the median region is reported (spread beside it)
  e2e        the same through the C interface with host (pinned) buffers: H2D of the source and
             D2H of the result inside the timed region; also upstream's literal three-call
             sequence with pinned and with pageable buffers
  roofline   the convolution kernel alone (CUDA events on the launching stream) against the
             ceiling of its own instruction measured in the same run (pipe_probe)
  cpu_baseline  the unmodified upstream library (bcast algorithm) on this machine's host cores,
             timed in a fresh process per executor the way upstream's perf tool does
  configs    the same figures, briefly, for the other benchmark layers (default: all five)

`--impl reference` times the upstream CPU library on the same layer (rank 0 only).
Inputs are synthetic (seeded), shapes and value distributions as the layer names say.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from xnor_nn_b200 import synth  # noqa: E402

# Cores this process may run on, taken before any OpenMP runtime is loaded: with OMP_PROC_BIND set
# the runtime pins the calling thread to one core, after which the affinity mask says "1".
HOST_CPUS = len(os.sched_getaffinity(0))
L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
MIN_TIMED_MS = 50.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="B", choices=list(synth.CONFIGS) + ["all"],
                    help="headline layer; `all` = B with every other layer in `configs`")
    ap.add_argument("--kernel", default="auto",
                    choices=["auto", "popc", "tcgen05_i8", "tcgen05_i8_rows"])
    ap.add_argument("--only", action="store_true", help="no `configs` array, headline layer only")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-probe", action="store_true", help="skip the pipe-rate probe")
    ap.add_argument("--passes", type=int, default=0,
                    help="profiler mode: run this many forward passes of the layer on device "
                         "tensors (optionally --minibatch images) and exit without timing")
    ap.add_argument("--minibatch", type=int, default=0, help="with --passes: images per pass")
    ap.add_argument("--chain", action="store_true",
                    help="time AlexNet conv3 -> conv4 -> conv5 layer by layer and as one chained "
                         "call (xnor_nn_b200_forward_chain), print one JSON line and exit")
    ap.add_argument("--pcie", action="store_true",
                    help="measure what the host delivers to the GPUs of this run: pinned "
                         "host-to-device, device-to-host and both at once, all ranks together; "
                         "print one JSON line and exit")
    ap.add_argument("--graph", action="store_true",
                    help="replay the step from CUDA graphs instead of calling the library")
    return ap.parse_args()


def conv_out(L):
    return ((L.ih + 2 * L.pw - L.kh) // L.sh + 1, (L.iw + 2 * L.pw - L.kw) // L.sw + 1)


def binary_ops(L, mb):
    oh, ow = conv_out(L)
    return 2.0 * mb * L.oc * oh * ow * L.ic * L.kh * L.kw


def pipe_probe():
    """Live ceilings of the candidate instruction paths (xnor_nn_b200/pipe_probe, built with the
    library): binary TOPS of the LOP3+POPC tile, of mma.sync b1 and of tcgen05.mma kind::i8."""
    exe = os.path.join(ROOT, "xnor_nn_b200", "pipe_probe")
    if not os.path.exists(exe):
        return None
    try:
        out = subprocess.run([exe], capture_output=True, text=True, timeout=120).stdout
        return json.loads(out.strip().splitlines()[-1])
    except (OSError, ValueError, IndexError, subprocess.TimeoutExpired):
        return None


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def captured_traffic(cfg, kernel_name):
    """DRAM bytes of one convolution launch taken from a profiler capture, if one is on record
    for this layer and kernel in bench_traffic.json (written beside the capture's summary);
    else None. Nothing is assumed: no record, no number."""
    path = os.path.join(ROOT, "bench_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f).get("%s/%s" % (cfg, kernel_name))
    except (OSError, ValueError):
        return None
    return rec


# ---- clocks ------------------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi sampled every 25 ms in the background; read-only."""
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def wait_live(self, seconds=5.0):
        """Blocks until the first sample has arrived (nvidia-smi needs a few hundred ms to start,
        more than the timed regions last), or `seconds` have passed."""
        t_end = time.time() + seconds
        while self.proc and not self.rows and time.time() < t_end and self.proc.poll() is None:
            time.sleep(0.005)

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        def parse_rows(rows):
            out = []
            for _, line in rows:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    out.append((float(p[2]), float(p[3]), p[5:9]))
                except ValueError:
                    pass
            return out
        inside = parse_rows([r for r in self.rows if t0 <= r[0] <= t1])
        window = "timed region"
        if not inside:
            inside = parse_rows([r for r in self.rows if t0 <= r[0] <= t1 + 0.15])
            window = "timed region + 150 ms (the region is shorter than the sampling period)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0,
                    "window": "nvidia-smi unavailable"}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for _, _, fl in inside for i in range(4)
                          if fl[i].lower().startswith("active")})
        return {"sm_mhz": float(np.median([r[0] for r in inside])),
                "sm_max_mhz": inside[0][1], "reasons": reasons, "samples": len(inside),
                "window": window}


# ---- reference arm / CPU baseline ----------------------------------------------------------------

def host_threads(want=None):
    """OpenMP threads the upstream library will use: all cores this process may run on, or
    `want`. (A launcher such as torchrun exports OMP_NUM_THREADS=1 for its workers; the CPU arm is
    meant to use the whole host, so the team size is set explicitly.)"""
    try:
        import ctypes
        omp = ctypes.CDLL("libgomp.so.1")
        if want is None:
            want = HOST_CPUS
        omp.omp_set_num_threads(want)
        return omp.omp_get_max_threads()
    except OSError:
        return os.cpu_count()


def upstream_times(L, cfg_name, mb, steps, warmup, threads=None):
    """Milliseconds per call of upstream's three per-minibatch executors (bcast algorithm) on
    `mb` images of layer L, measured the way upstream's perf tool measures them
    (test/perf/test_simple_net.cpp:32-60,130-144): every timed call is preceded by a pass that
    dirties a buffer larger than the last-level cache slices the call will use, and the clock
    runs around the call only. Returns (dict of medians in ms, threads used)."""
    import ctypes as C
    from oracle.pyoracle import UpstreamRef, UpstreamConv
    ref = UpstreamRef()
    used = host_threads(threads)
    src, w = synth.make_inputs(cfg_name, mb=mb)
    c = UpstreamConv()
    assert ref.lib.xnor_nn_init_convolution(C.byref(c), 1, 0, 2, 0, mb, L.oc, L.ic, L.ih, L.iw,
                                            L.kh, L.kw, L.sh, L.sw, L.ph, L.pw) == 0
    res = (C.c_void_p * 9)()
    assert ref.lib.xnor_nn_allocate_resources(C.byref(c), res) == 0
    dst = np.empty(mb * c.oc * c.oh * c.ow, np.float32)
    res[0], res[1], res[2] = src.ctypes.data, w.ctypes.data, dst.ctypes.data
    assert c.binarize_weights(C.addressof(c), res) == 0
    trash = np.zeros(64 << 20, np.uint8)  # upstream dirties 16 MB; server L3s are larger
    out = {}
    for name in ("binarize_data", "calculate_k", "forward"):
        ex = getattr(c, name)
        times = []
        for i in range(warmup + steps):
            trash += 1
            t0 = time.perf_counter()
            assert ex(C.addressof(c), res) == 0
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
        out[name] = float(np.median(times)) * 1e3
    ref.lib.xnor_nn_free_resources(res)
    ref.lib.xnor_nn_destroy_convolution(C.byref(c))
    return out, used


def reference_line(args, cfg_name, L):
    """The JSON object of the reference arm for one layer (upstream library, all host threads)."""
    from oracle.pyoracle import UpstreamRef
    if not UpstreamRef.available():
        return {"impl": "reference",
                "unavailable": "oracle/_ref/libxnor_nn_ref.so was not built"}
    # Bounded sample: the whole minibatch unless that would take minutes.
    probe, _ = upstream_times(L, cfg_name, min(L.mb, 8), 1, 1)
    per_image = sum(probe.values()) * 1e-3 / min(L.mb, 8)
    mb = L.mb
    while mb > 8 and per_image * mb * (args.steps + max(1, args.warmup)) > 100.0:
        mb //= 2
    t, threads = upstream_times(L, cfg_name, mb, args.steps, max(1, args.warmup))
    scale = L.mb / mb
    ms = sum(t.values()) * scale
    tops = binary_ops(L, L.mb) / (ms * 1e-3) / 1e12
    sample = "%d of %d images per step, %d steps" % (mb, L.mb, args.steps)
    return {
        "impl": "reference", "metric": "effective_binary_tops", "value": tops, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": max(1, args.warmup),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": L.name, "algorithm": "upstream bcast, XNOR_NN_ISA=2",
                   "sample": sample, "omp_threads": threads,
                   "omp_proc_bind": os.environ.get("OMP_PROC_BIND", "unset"),
                   "protocol": "per executor, cache dirtied before every timed call, median"},
        "executors_ms": {k: v * scale for k, v in t.items()},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "reference",
                         "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}


def run_reference(args, cfg_name, L, rank):
    if rank != 0:
        return
    print(json.dumps(reference_line(args, cfg_name, L)))


def cpu_baseline_subprocess(cfg_name, steps):
    """The reference arm in a process of its own (no CUDA context, no torch threads, threads
    bound to neighbouring cores) so that it measures what `--impl reference` measures."""
    env = dict(os.environ)
    env.pop("OMP_NUM_THREADS", None)
    env.setdefault("OMP_PROC_BIND", "close")
    env.setdefault("XNOR_NN_ISA", "2")
    try:
        out = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference",
                              "--config", cfg_name, "--steps", str(steps), "--warmup", "2"],
                             capture_output=True, text=True, timeout=600, env=env).stdout
        d = json.loads(out.strip().splitlines()[-1])
    except (OSError, ValueError, IndexError, subprocess.TimeoutExpired):
        return None
    if "unavailable" in d:
        return None
    return {"value": d["value"], "unit": "TOPS", "cores": d["cpu_baseline"]["cores"],
            "kind": "reference", "sample": d["cpu_baseline"]["sample"],
            "ms_per_step": d["ms_per_step"], "executors_ms": d["executors_ms"],
            "omp_proc_bind": d["config"]["omp_proc_bind"], "process": "fresh subprocess"}


# ---- our arm -------------------------------------------------------------------------------------

class Layer:
    """One benchmark layer on this rank's GPU: its slice of the minibatch, rotating device
    tensors, and the timing helpers."""

    def __init__(self, xb, torch, cfg_name, kernel, rank, world):
        from xnor_nn_b200.sharding import shard_range
        self.xb, self.torch, self.cfg = xb, torch, cfg_name
        L = self.L = synth.CONFIGS[cfg_name]
        first, last = shard_range(L.mb, rank, world)
        self.first, self.mb = first, last - first
        self.oh, self.ow = conv_out(L)
        self.stream = torch.cuda.current_stream()
        self.kernel_name = None
        self.n_src = self.n_dst = self.step_bytes = self.sets = 0
        if self.mb == 0:  # more GPUs than images: this rank only keeps the others company
            self.conv = None
            return
        self.src_np, self.w_np = synth.make_inputs(cfg_name, mb=self.mb, first_image=first)
        self.conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, self.mb, L.oc,
                                   L.ic, L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw,
                                   self.w_np, kernel=kernel)
        self.kernel_name = xb.KERNEL_NAMES[self.conv.kernel]
        self.conv.set_stream(self.stream.cuda_stream)
        # Rotating device buffers: consecutive steps touch different tensors and one full
        # rotation exceeds L2 several times over, so no step finds its input or output cached.
        self.n_src, self.n_dst = self.src_np.size, self.mb * L.oc * self.oh * self.ow
        self.step_bytes = 4 * (self.n_src + self.n_dst)
        self.sets = min(48, max(2, int(np.ceil(3.2 * L2_BYTES / self.step_bytes)) + 1))
        self.d_src = [torch.from_numpy(self.src_np).cuda() for _ in range(self.sets)]
        self.d_dst = [torch.empty(self.n_dst, dtype=torch.float32, device="cuda")
                      for _ in range(self.sets)]

    def step(self, i):
        if self.conv is not None:
            self.conv.forward(self.d_src[i % self.sets], self.d_dst[i % self.sets])

    def conv_only(self, i):
        import ctypes as C
        if self.conv is None:
            return
        xb = self.xb
        self.conv._set(xb.SLOT_USER_DST, self.d_dst[i % self.sets])
        st = self.conv.c.forward(C.addressof(self.conv.c), self.conv.res)
        assert st == xb.SUCCESS, xb.last_error()

    def bin_only(self, i):
        import ctypes as C
        if self.conv is None:
            return
        xb = self.xb
        self.conv._set(xb.SLOT_USER_SRC, self.d_src[i % self.sets])
        st = xb.lib().xnor_nn_b200_binarize(C.byref(self.conv.c), self.conv.res)
        assert st == xb.SUCCESS, xb.last_error()

    def region_ms(self, fn, n, offset=0):
        """Device time of n consecutive calls of fn, CUDA events on the launching stream."""
        torch = self.torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(self.stream)
        for i in range(n):
            fn(offset + i)
        b.record(self.stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    def timed(self, fn, n, min_ms=10.0):
        """Median milliseconds per call over regions of n calls, at least min_ms timed."""
        for i in range(3):
            fn(i)
        self.torch.cuda.synchronize()
        per, total, k = [], 0.0, 0
        while total < min_ms or len(per) < 3:
            ms = self.region_ms(fn, n, k * n)
            per.append(ms / n)
            total += ms
            k += 1
            if k >= 200:
                break
        return float(np.median(per))

    def parity_ok(self, oracle_mod):
        """First and last image of this rank's slice against the CPU oracle (outside any timed
        region): integer-exact results scaled in upstream's order, so the floats must agree to
        1e-4 relative."""
        torch = self.torch
        L = self.L
        self.step(0)
        torch.cuda.synchronize()
        got = self.d_dst[0].cpu().numpy()
        per = L.oc * self.oh * self.ow
        orc = oracle_mod.Oracle()
        for img in sorted({0, self.mb - 1}):
            s = oracle_mod.Shape.make(1, L.oc, L.ic, L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw)
            want = orc.convolution(s, self.src_np[img:img + 1], self.w_np)["dst"]
            err = np.abs(got[img * per:(img + 1) * per] - want)
            if not np.all(err <= 1e-4 * np.abs(want)):
                return False
        return True

    def close(self):
        if self.conv is not None:
            self.conv.close()
        self.d_src = self.d_dst = None
        self.torch.cuda.empty_cache()


def measure_layer(xb, torch, args, cfg_name, kernel, rank, world, dist, probe, brief):
    """All figures of one layer. `brief` (the `configs` entries) leaves out the literal
    three-call sequence, the clocks and the CUDA-graph option."""
    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    lay = Layer(xb, torch, cfg_name, kernel, rank, world)
    L, mb = lay.L, lay.mb
    steps = args.steps if not brief else max(20, min(args.steps, 100))

    # parity of this rank's slice, outside the timed regions
    ok = True
    if mb > 0:
        from oracle import pyoracle  # the checker, outside every timed region
        ok = lay.parity_ok(pyoracle)
    if dist is not None:
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = bool(t.item())

    graphs = None
    launches_per_step = None
    step = lay.step
    if args.graph and not brief:
        for i in range(2):
            lay.step(i)
        torch.cuda.synchronize()
        graphs = []
        side = torch.cuda.Stream()
        lay.conv.set_stream(side.cuda_stream)  # before capture starts: switching synchronises
        for k in range(lay.sets):
            g = torch.cuda.CUDAGraph()
            before = xb.kernel_launches()
            with torch.cuda.graph(g, stream=side):
                lay.conv.forward(lay.d_src[k], lay.d_dst[k])
            launches_per_step = xb.kernel_launches() - before
            graphs.append(g)
        lay.conv.set_stream(lay.stream.cuda_stream)

        def step(i):
            graphs[i % lay.sets].replay()

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 and not brief else None
    if sampler:
        sampler.wait_live()
    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    # Regions of exactly `steps` steps, each bracketed by a barrier and a device synchronise and
    # timed as the slowest rank, repeated until MIN_TIMED_MS have been timed.
    launches0 = xb.kernel_launches()
    t_wall0 = time.time()
    regions, total = [], 0.0
    while (total < MIN_TIMED_MS or len(regions) < 3) and len(regions) < 400:
        barrier()
        ms = max_over_ranks(lay.region_ms(step, steps, len(regions) * steps))
        regions.append(ms / steps)
        total += ms
    t_wall1 = time.time()
    barrier()
    launches = xb.kernel_launches() - launches0
    if graphs is not None:
        launches = launches_per_step * steps * len(regions)
    ms_step = float(np.median(regions))
    value = binary_ops(L, L.mb) / (ms_step * 1e-3) / 1e12

    # ---- the two kernels alone, same rotation; the slowest rank's figures are reported (with
    # more GPUs than images some ranks, possibly rank 0, have nothing to do) -------------------
    if lay.conv is not None:
        lay.conv._set(xb.SLOT_USER_SRC, lay.d_src[0])
    n_k = max(20, min(steps, 200))
    conv_ms = max_over_ranks(lay.timed(lay.conv_only, n_k) if lay.conv is not None else 0.0)
    bin_ms = max_over_ranks(lay.timed(lay.bin_only, n_k) if lay.conv is not None else 0.0)
    mb_max = int(max_over_ranks(float(mb)))
    if dist is not None:
        names = [None] * world
        dist.all_gather_object(names, lay.kernel_name)
        lay.kernel_name = next(n for n in names if n)
    n_src_max = lay.n_src if mb == mb_max else mb_max * L.ic * L.ih * L.iw
    # compulsory bytes of the packing pass: 4 B per source element in, 1 B (tensor-core family)
    # or 1 bit (integer-pipe family) per element out, plus the mean-|x| map
    tc = (lay.kernel_name or "tcgen05").startswith("tcgen05")
    bin_bytes = 4.0 * n_src_max + (n_src_max if tc else n_src_max / 8.0) + 4.0 * mb_max * L.ih * L.iw
    pk, pk_kind = peaks()
    conv_tops = binary_ops(L, mb_max) / (conv_ms * 1e-3) / 1e12
    if tc:
        peak = probe.get("tcgen05_i8_tops") if probe else None
        peak_note = "tcgen05.mma kind::i8 ceiling measured in this run (pipe_probe)"
        bound = "tensor"
    else:
        peak = probe.get("popc_binary_tops") if probe else None
        peak_note = "LOP3+POPC ceiling measured in this run (pipe_probe)"
        bound = "int_pipe"
    alt_peak = 2.0 * pk["bf16_tflops"] if tc else None
    traffic = captured_traffic(cfg_name, lay.kernel_name) if world == 1 else None
    roofline = {"kernel": "conv_" + lay.kernel_name, "bound": bound, "achieved": conv_tops,
                "peak": peak, "unit": "TFLOP/s", "frac": (conv_tops / peak) if peak else None,
                "traffic": traffic["bytes"] if traffic else None,
                "traffic_source": traffic.get("source") if traffic else None,
                "peak_source": peak_note, "ms": conv_ms,
                "timing": "launches issued back to back on one stream, CUDA events around the "
                          "sequence, milliseconds per launch (includes what lies between launches)",
                "frac_of_2x_bf16_%s" % pk_kind: (conv_tops / alt_peak) if alt_peak else None,
                "binarize": {"kernel": "sign-pack with the mean-|x| map (the pass the step runs)",
                             "bound": "hbm", "achieved": bin_bytes / (bin_ms * 1e-3) / 1e9,
                             "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": bin_bytes / (bin_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                             "ms": bin_ms, "peak_source": pk_kind,
                             "bytes": "fp32 source read once + packed activations and map written"}}

    # ---- end to end: host buffers through the C interface -----------------------------------
    if lay.conv is not None:
        lay.conv.synchronize()
        h_src = torch.from_numpy(lay.src_np).pin_memory()
        h_dst = torch.empty(lay.n_dst, dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(steps, 20))

    def e2e_ms(which, src, dst):
        call = getattr(lay.conv, which) if lay.conv is not None else (lambda a, b: None)
        for _ in range(2):
            call(src, dst)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(lay.stream)
        for _ in range(e2e_steps):
            call(src, dst)  # returns when dst is complete
        b.record(lay.stream)
        torch.cuda.synchronize()
        barrier()
        return max_over_ranks(a.elapsed_time(b)) / e2e_steps

    if lay.conv is None:
        h_src = h_dst = None
    one_call = e2e_ms("forward", h_src, h_dst)
    e2e = {"value": binary_ops(L, L.mb) / (one_call * 1e-3) / 1e12, "unit": "TOPS",
           "h2d_bytes_per_step": 4 * lay.n_src, "d2h_bytes_per_step": 4 * lay.n_dst,
           "ms_per_step": one_call, "call": "xnor_nn_b200_forward (host pointers, pinned)"}
    if not brief:
        e2e["three_calls_pinned_ms"] = e2e_ms("forward_stepwise", h_src, h_dst)
        p_src = lay.src_np if lay.conv is not None else None
        p_dst = np.empty(lay.n_dst, np.float32) if lay.conv is not None else None
        e2e["three_calls_pageable_ms"] = e2e_ms("forward_stepwise", p_src, p_dst)
        e2e["one_call_pageable_ms"] = e2e_ms("forward", p_src, p_dst)
        e2e["three_calls"] = ("binarize_data, calculate_k, forward through the executor pointers, "
                              "as upstream's wrapper issues them")

    clocks = None
    if sampler:
        sampler.stop()
        clocks = sampler.summary(t_wall0, t_wall1)

    line = {
        "metric": "effective_binary_tops", "value": value, "unit": "TOPS", "n_gpus": world,
        "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
        "ms_per_step_min": float(np.min(regions)), "ms_per_step_max": float(np.max(regions)),
        "timed_regions": len(regions), "timed_ms": total,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "s8" if tc else "u32", "data": "synthetic",
        "config": {"workload": L.name, "minibatch": L.mb, "images_per_gpu": mb_max,
                   "kernel": lay.kernel_name, "parallelism": "minibatch slices x%d" % world,
                   "l2": ("inputs larger than L2: %d rotating tensor sets of %.1f MB"
                          if lay.sets * lay.step_bytes > 2 * L2_BYTES else
                          "%d rotating tensor sets of %.2f MB: smaller than L2, a layer this "
                          "small is bound by latency, not by memory")
                         % (lay.sets, lay.step_bytes / 1e6),
                   "launch": "cuda graph replay, one graph per tensor set"
                             if graphs is not None else "plain calls"},
        "parity_checked": ok,
        "roofline": roofline, "e2e": e2e, "clocks": clocks, "gpu_launches": int(launches)}
    lay.close()
    return line


def chain_line(xb, torch, mb, reps):
    """AlexNet's conv3 -> conv4 -> conv5 (13x13, 3x3, pad 1: 256 -> 384 -> 256 -> 256 channels)
    layer by layer and as one chained call, tensors resident on the device, microseconds per
    pass (six rotating tensor sets so that a pass does not find its inputs in L2)."""
    channels = (256, 384, 256, 256)
    convs = []
    for i in range(3):
        ic, oc = channels[i], channels[i + 1]
        w = synth.normal(0xBEEF0000 + i, oc * ic * 9, 0.05)
        convs.append(xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, mb, oc, ic, 13,
                                    13, 3, 3, 1, 1, 1, 1, w))
    stream = torch.cuda.current_stream().cuda_stream
    for cv in convs:
        cv.set_stream(stream)
    sets = 6
    bufs = [[torch.randn(mb * c * 169, device="cuda") for c in channels] for _ in range(sets)]

    def timed(fn):
        for i in range(30):
            fn(bufs[i % sets])
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(reps):
            fn(bufs[i % sets])
        t1.record()
        torch.cuda.synchronize()
        return round(t0.elapsed_time(t1) / reps * 1e3, 1)

    def separate(n):
        def run(b):
            for i in range(n):
                convs[i].forward(b[i], b[i + 1])
        return run

    def chained(n):
        return lambda b: xb.forward_chain(convs[:n], b[0], b[n])

    print(json.dumps({
        "chain": "alexnet conv3 -> conv4 -> conv5", "minibatch": mb, "reps": reps,
        "unit": "us per pass",
        "conv3_conv4": {"layer_by_layer": timed(separate(2)), "chained": timed(chained(2))},
        "conv3_conv4_conv5": {"layer_by_layer": timed(separate(3)), "chained": timed(chained(3))}}))
    for cv in convs:
        cv.close()


def pcie_line(torch, dist, rank, world):
    """Pinned-memory copy rates with every rank of the run copying at the same time: the floor
    under the end-to-end figure, whose every step moves its slice up and its results down."""
    mb = 64
    h_up = torch.empty(mb << 20, dtype=torch.uint8).pin_memory()
    h_dn = torch.empty(mb << 20, dtype=torch.uint8).pin_memory()
    d_up = torch.empty(mb << 20, dtype=torch.uint8, device="cuda")
    d_dn = torch.empty(mb << 20, dtype=torch.uint8, device="cuda")
    s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def gbs(up, down, reps=8):
        rates = []
        for _ in range(3):
            barrier()
            t0 = time.perf_counter()
            for _ in range(reps):
                if up:
                    with torch.cuda.stream(s_up):
                        d_up.copy_(h_up, non_blocking=True)
                if down:
                    with torch.cuda.stream(s_dn):
                        h_dn.copy_(d_dn, non_blocking=True)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            rates.append((up + down) * reps * (mb << 20) / dt / 1e9)
        return float(np.median(rates))

    mine = [gbs(1, 0), gbs(0, 1), gbs(1, 1)]
    rows = [mine]
    if dist is not None:
        rows = [None] * world
        dist.all_gather_object(rows, mine)
    if rank == 0:
        a = np.array(rows)
        print(json.dumps({
            "pcie": "pinned host memory, %d MB per copy, all %d ranks at once" % (mb, world),
            "n_gpus": world, "unit": "GB/s",
            "per_rank": {"h2d": a[:, 0].round(1).tolist(), "d2h": a[:, 1].round(1).tolist(),
                         "both_directions": a[:, 2].round(1).tolist()},
            "aggregate": {"h2d": float(a[:, 0].sum()), "d2h": float(a[:, 1].sum()),
                          "both_directions": float(a[:, 2].sum())},
            "slowest_rank": {"h2d": float(a[:, 0].min()), "d2h": float(a[:, 1].min()),
                             "both_directions": float(a[:, 2].min())}}))


def run_ours(args, rank, world, local_rank):
    import torch
    import xnor_nn_b200 as xb

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    kernel = {"auto": xb.KERNEL_AUTO, "popc": xb.KERNEL_POPC, "tcgen05_i8": xb.KERNEL_TCGEN05_I8,
              "tcgen05_i8_rows": xb.KERNEL_TCGEN05_I8_ROWS}[args.kernel]
    head = "B" if args.config == "all" else args.config
    if args.passes:
        # a handful of launches for a profiler: few warm-ups, nothing else on the device
        L = synth.CONFIGS[head]
        mb = args.minibatch or L.mb
        src, w = synth.make_inputs(head, mb=mb)
        conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, mb, L.oc, L.ic, L.ih,
                              L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w, kernel=kernel)
        d_src = torch.from_numpy(src).cuda()
        d_dst = torch.empty(int(np.prod(conv.out_shape)), device="cuda")
        for _ in range(args.passes):
            conv.forward(d_src, d_dst)
        conv.synchronize()
        print("ok %s mb=%d passes=%d" % (xb.KERNEL_NAMES[conv.kernel], mb, args.passes))
        conv.close()
        return
    if args.chain:
        chain_line(xb, torch, args.minibatch or 256, max(20, min(args.steps, 200)))
        return
    if args.pcie:
        pcie_line(torch, dist, rank, world)
        if dist is not None:
            dist.destroy_process_group()
        return
    others = [] if args.only else [c for c in synth.CONFIGS if c != head]
    probe = pipe_probe() if rank == 0 and not args.no_probe else None
    if dist is not None:  # every rank computes the fraction of the same ceiling
        box = [probe]
        dist.broadcast_object_list(box, src=0)
        probe = box[0]

    line = measure_layer(xb, torch, args, head, kernel, rank, world, dist, probe, brief=False)
    line["roofline"]["pipe_probe"] = probe
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_subprocess(head, 10)
    else:
        line["cpu_baseline"] = None
    configs = []
    for cfg in others:
        d = measure_layer(xb, torch, args, cfg, kernel, rank, world, dist, probe, brief=True)
        entry = {"config": cfg, "workload": d["config"]["workload"],
                 "images_per_gpu": d["config"]["images_per_gpu"], "kernel": d["config"]["kernel"],
                 "ms_per_step": d["ms_per_step"], "value": d["value"], "unit": "TOPS",
                 "conv_ms": d["roofline"]["ms"], "conv_tops": d["roofline"]["achieved"],
                 "conv_frac": d["roofline"]["frac"], "binarize_ms": d["roofline"]["binarize"]["ms"],
                 "binarize_frac": d["roofline"]["binarize"]["frac"],
                 "e2e_ms": d["e2e"]["ms_per_step"], "parity_checked": d["parity_checked"]}
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline_subprocess(cfg, 3)
            entry["cpu_ms"] = cpu["ms_per_step"] if cpu else None
            entry["cpu_cores"] = cpu["cores"] if cpu else None
        configs.append(entry)
    line["configs"] = configs
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        os.environ.setdefault("OMP_PROC_BIND", "close")  # read by libgomp when it is loaded
        os.environ.setdefault("XNOR_NN_ISA", "2")
        head = "B" if args.config == "all" else args.config
        run_reference(args, head, synth.CONFIGS[head], rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
