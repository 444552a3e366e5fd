"""Benchmark of the binary-convolution path: AlexNet conv4, minibatch 256, on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config A..E] [--kernel auto|popc|mma_b1|tcgen05_i8]

A step is one forward pass of the layer (sign-pack + mean-|x| map, K box filter, XNOR/popcount
convolution with the alpha*K epilogue) over the whole minibatch; with N GPUs the minibatch is
split into N contiguous slices, one process per GPU, no collective on the data path (strong
scaling: the total batch stays 256). Rank 0 prints one JSON line.

  value      effective binary TOPS = 2*MB*OC*OH*OW*IC*KH*KW / time, tensors resident in HBM
  e2e        the same through the C interface with host (pinned) buffers: H2D of the source
             and D2H of the result inside the timed region
  roofline   the convolution kernel alone, CUDA events on the launching stream
  cpu_baseline  the unmodified upstream library (bcast algorithm) on this machine's host cores

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

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="B", choices=list(synth.CONFIGS))
    ap.add_argument("--kernel", default="auto", choices=["auto", "popc", "mma_b1", "tcgen05_i8"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0,
                    help="budget of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-probe", action="store_true", help="skip the pipe-rate probe")
    ap.add_argument("--graph", action="store_true",
                    help="replay the step from CUDA graphs instead of calling the library")
    return ap.parse_args()


def binary_ops(L, mb):
    return 2.0 * mb * L.oc * conv_out(L)[0] * conv_out(L)[1] * L.ic * L.kh * L.kw


def conv_out(L):
    return ((L.ih + 2 * L.pw - L.kh) // L.sh + 1, (L.iw + 2 * L.pw - L.kw) // L.sw + 1)


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


# DRAM bytes of one convolution launch on the benchmark layer, from the ncu capture summarised
# in profiles/ (dram__bytes_read.sum + dram__bytes_write.sum): the packed operands are read once,
# the 44 MB result is still in L2 when the kernel ends.
NCU_CONV_TRAFFIC = {("B", "tcgen05_i8"): 20.37e6 + 0.31e6}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


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
        inside = parse_rows([r for r in self.rows if t0 <= r[0] <= t1 + 0.15])
        window = "timed region"
        if not inside:
            inside = parse_rows(self.rows)
            window = "whole run (timed region shorter than the sampling period)"
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

def upstream_forward_seconds(L, mb, budget_s, steps=None, warmup=1, threads=None):
    """Seconds per forward pass (binarize_data + calculate_k + forward, what upstream's
    Convolution::forward runs) of the unmodified upstream library, bcast algorithm, all host
    threads, on `mb` images of layer L. Timed like upstream's perf harness
    (test/perf/test_simple_net.cpp:39-60): wall clock around the executor calls."""
    import ctypes as C
    from oracle.pyoracle import UpstreamRef, UpstreamConv
    ref = UpstreamRef()
    host_threads(threads)
    cfg_name = [k for k, v in synth.CONFIGS.items() if v.name == L.name][0]
    src, w = synth.make_inputs(cfg_name, mb=mb)
    c = UpstreamConv()
    assert ref.lib.xnor_nn_init_convolution(C.byref(c), 1, 0, 2, 0, mb, L.oc, L.ic, L.ih, L.iw,
                                            L.kh, L.kw, L.sh, L.sw, L.ph, L.pw) == 0
    res = (C.c_void_p * 9)()
    assert ref.lib.xnor_nn_allocate_resources(C.byref(c), res) == 0
    dst = np.empty(mb * c.oc * c.oh * c.ow, np.float32)
    res[0], res[1], res[2] = src.ctypes.data, w.ctypes.data, dst.ctypes.data
    assert c.binarize_weights(C.addressof(c), res) == 0

    def one():
        t0 = time.perf_counter()
        for ex in (c.binarize_data, c.calculate_k, c.forward):
            assert ex(C.addressof(c), res) == 0
        return time.perf_counter() - t0

    for _ in range(warmup):
        first = one()
    times = []
    if steps is None:
        steps = max(1, min(50, int(budget_s / max(first, 1e-6))))
    for _ in range(steps):
        times.append(one())
    ref.lib.xnor_nn_free_resources(res)
    ref.lib.xnor_nn_destroy_convolution(C.byref(c))
    return float(np.sum(times)), steps


def host_threads(want=None):
    """OpenMP threads the upstream library will use: all cores this process may run on, or
    `want`. (A launcher such as torchrun exports OMP_NUM_THREADS=1 for its workers; the CPU arm is
    meant to use the whole host, so the team size is set explicitly.)"""
    try:
        import ctypes
        omp = ctypes.CDLL("libgomp.so.1")
        if want is None:
            want = len(os.sched_getaffinity(0))
        omp.omp_set_num_threads(want)
        return omp.omp_get_max_threads()
    except OSError:
        return os.cpu_count()


def run_reference(args, L, rank):
    if rank != 0:
        return
    from oracle.pyoracle import UpstreamRef
    if not UpstreamRef.available():
        print(json.dumps({"impl": "reference",
                          "unavailable": "oracle/_ref/libxnor_nn_ref.so was not built"}))
        return
    # Bounded sample: the full layer is ~0.1-1 s per pass on a server CPU, so each step is the
    # whole minibatch unless that would take minutes.
    probe, _ = upstream_forward_seconds(L, min(L.mb, 8), 0, steps=1, warmup=1)
    per_image = probe / min(L.mb, 8)
    budget = 150.0
    mb = L.mb
    while mb > 8 and per_image * mb * (args.steps + args.warmup) > budget:
        mb //= 2
    total, steps = upstream_forward_seconds(L, mb, 0, steps=args.steps, warmup=max(1, args.warmup))
    sec = total / steps
    tops = binary_ops(L, mb) / sec / 1e12
    threads = host_threads()
    sample = "%d of %d images per step, %d steps" % (mb, L.mb, steps)
    print(json.dumps({
        "impl": "reference", "metric": "effective_binary_tops", "value": tops, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": steps, "warmup": max(1, args.warmup),
        "ms_per_step": sec * 1e3 * (L.mb / mb), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": L.name, "algorithm": "upstream bcast, XNOR_NN_ISA=2",
                   "sample": sample},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "reference",
                         "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# ---- our arm -------------------------------------------------------------------------------------

def run_ours(args, L, rank, world, local_rank):
    import torch
    import xnor_nn_b200 as xb

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

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

    from xnor_nn_b200.sharding import shard_range
    first, last = shard_range(L.mb, rank, world)
    mb = last - first
    oh, ow = conv_out(L)
    kernel = {"auto": xb.KERNEL_AUTO, "popc": xb.KERNEL_POPC, "mma_b1": xb.KERNEL_MMA_B1,
              "tcgen05_i8": xb.KERNEL_TCGEN05_I8}[args.kernel]

    src_np, w_np = synth.make_inputs(args.config, mb=mb, first_image=first)
    conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, mb, L.oc, L.ic, L.ih,
                          L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w_np, kernel=kernel)
    kernel_name = xb.KERNEL_NAMES[conv.kernel]
    stream = torch.cuda.current_stream()
    conv.set_stream(stream.cuda_stream)

    # Rotating device buffers: consecutive steps touch different tensors and one full rotation
    # exceeds L2 several times over, so no step finds its input or output cached.
    n_src, n_dst = src_np.size, mb * L.oc * oh * ow
    step_bytes = 4 * (n_src + n_dst)
    sets = max(2, int(np.ceil(3.2 * L2_BYTES / step_bytes)) + 1)
    d_src = [torch.from_numpy(src_np).cuda() for _ in range(sets)]
    d_dst = [torch.empty(n_dst, dtype=torch.float32, device="cuda") for _ in range(sets)]

    def eager_step(i):
        conv.forward(d_src[i % sets], d_dst[i % sets])

    # The step is two kernel launches behind a C call. --graph replays it from a CUDA graph (one
    # per tensor set, captured once), which takes the host out of the loop; the same kernels run
    # either way. Plain calls are the default because they are faster here: consecutive launches
    # of one stream overlap their set-up with the predecessor's tail, consecutive graph launches
    # do not (54.3 vs 55.4 us per step on conv4).
    graphs = None
    launches_per_step = None
    if args.graph:
        for i in range(2):
            eager_step(i)
        torch.cuda.synchronize()
        graphs = []
        side = torch.cuda.Stream()
        conv.set_stream(side.cuda_stream)  # before capture starts: switching streams synchronises
        for k in range(sets):
            g = torch.cuda.CUDAGraph()
            before = xb.kernel_launches()
            with torch.cuda.graph(g, stream=side):
                conv.forward(d_src[k], d_dst[k])
            launches_per_step = xb.kernel_launches() - before
            graphs.append(g)
        conv.set_stream(stream.cuda_stream)

    def step(i):
        if graphs is not None:
            graphs[i % sets].replay()
        else:
            eager_step(i)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    launches0 = xb.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    t_wall1 = time.time()
    launches = xb.kernel_launches() - launches0
    if graphs is not None:
        launches = launches_per_step * args.steps  # kernel nodes replayed inside the timed region
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    value = binary_ops(L, L.mb) / (ms_step * 1e-3) / 1e12

    # ---- the dominant kernel alone (convolution), same rotation -----------------------------
    import ctypes as C
    conv._set(xb.SLOT_USER_SRC, d_src[0])

    def conv_only(i):
        conv._set(xb.SLOT_USER_DST, d_dst[i % sets])
        st = conv.c.forward(C.addressof(conv.c), conv.res)
        assert st == xb.SUCCESS, xb.last_error()

    def bin_only(i):
        conv._set(xb.SLOT_USER_SRC, d_src[i % sets])
        st = conv.c.binarize_data(C.addressof(conv.c), conv.res)
        assert st == xb.SUCCESS, xb.last_error()

    def timed(fn, n):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(n):
            fn(i)
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    n_k = max(20, min(args.steps, 200))
    conv_ms = timed(conv_only, n_k)
    bin_ms = timed(bin_only, n_k)
    # compulsory bytes of the packing pass: 4 B per source element in, 1 B (tensor-core family)
    # or 1 bit (bit families) per element out
    bin_bytes = 4.0 * n_src + (n_src if kernel_name == "tcgen05_i8" else n_src / 8.0)
    pk, pk_kind = peaks()
    probe = pipe_probe() if rank == 0 and not args.no_probe else None
    conv_tops = binary_ops(L, mb) / (conv_ms * 1e-3) / 1e12
    probe_peak = None
    if kernel_name == "tcgen05_i8":
        # 8-bit operands issue at twice the 16-bit rate on the same tensor pipe
        peak = 2.0 * pk["bf16_tflops"]
        peak_note = "2 x %s bf16 dense burst (8-bit operands)" % pk_kind
        bound = "tensor"
        probe_peak = probe.get("tcgen05_i8_tops") if probe else None
    else:
        key = "mma_b1_binary_tops" if kernel_name == "mma_b1" else "popc_binary_tops"
        peak = probe.get(key) if probe else None
        peak_note = "pipe_probe, measured in this run (no MEASURED_PEAKS entry for this pipe)"
        bound = "tensor" if kernel_name == "mma_b1" else "int_pipe"
        probe_peak = peak
    roofline = {"kernel": "conv_" + kernel_name, "bound": bound, "achieved": conv_tops,
                "peak": peak, "unit": "TFLOP/s", "frac": (conv_tops / peak) if peak else None,
                "traffic": NCU_CONV_TRAFFIC.get((args.config, kernel_name)) if world == 1 else None,
                "peak_source": peak_note, "ms": conv_ms,
                "frac_of_probe_peak": (conv_tops / probe_peak) if probe_peak else None,
                "pipe_probe": probe,
                "binarize": {"bound": "hbm", "achieved": bin_bytes / (bin_ms * 1e-3) / 1e9,
                             "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": bin_bytes / (bin_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                             "ms": bin_ms, "peak_source": pk_kind,
                             "bytes": "fp32 source read once + packed activations written"}}

    # ---- end to end: host buffers through the C interface -----------------------------------
    conv.synchronize()
    h_src = torch.from_numpy(src_np).pin_memory()
    h_dst = torch.empty(n_dst, dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(args.steps, 30))
    for _ in range(3):
        conv.forward(h_src, h_dst)
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(e2e_steps):
        conv.forward(h_src, h_dst)  # returns when h_dst is complete
    b.record(stream)
    torch.cuda.synchronize()
    barrier()
    e2e_ms = max_over_ranks(a.elapsed_time(b)) / e2e_steps
    e2e = {"value": binary_ops(L, L.mb) / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS",
           "h2d_bytes_per_step": 4 * n_src, "d2h_bytes_per_step": 4 * n_dst, "ms_per_step": e2e_ms,
           "call": "xnor_nn_b200_forward (host pointers, pinned)"}

    clocks = None
    if sampler:
        time.sleep(0.12)
        sampler.stop()
        clocks = sampler.summary(t_wall0, t_wall1)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle.pyoracle import UpstreamRef
        if UpstreamRef.available():
            total, steps = upstream_forward_seconds(L, L.mb, args.cpu_seconds)
            cpu = {"value": binary_ops(L, L.mb) / (total / steps) / 1e12, "unit": "TOPS",
                   "cores": host_threads(), "kind": "reference",
                   "ms_per_step": total / steps * 1e3,
                   "sample": "full minibatch (%d images), %d passes, upstream bcast, "
                             "XNOR_NN_ISA=2" % (L.mb, steps)}
            # the same library on one thread, on a few images (it scales with the image count)
            few = min(L.mb, 8)
            t1, n1 = upstream_forward_seconds(L, few, 0, steps=2, warmup=1, threads=1)
            cpu["one_thread"] = {"value": binary_ops(L, few) / (t1 / n1) / 1e12, "unit": "TOPS",
                                 "ms_per_step": t1 / n1 * 1e3 * (L.mb / few),
                                 "sample": "%d of %d images, scaled" % (few, L.mb)}
            host_threads()

    if rank == 0:
        print(json.dumps({
            "metric": "effective_binary_tops", "value": value, "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "s8" if kernel_name == "tcgen05_i8" else "u32", "data": "synthetic",
            "config": {"workload": L.name, "minibatch": L.mb, "images_per_gpu": mb,
                       "kernel": kernel_name, "parallelism": "minibatch slices x%d" % world,
                       "l2": "inputs larger than L2: %d rotating tensor sets of %.1f MB"
                             % (sets, step_bytes / 1e6),
                       "launch": "cuda graph replay, one graph per tensor set"
                                 if graphs is not None else "plain calls"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": int(launches)}))
    conv.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    L = synth.CONFIGS[args.config]
    if args.impl == "reference":
        run_reference(args, L, rank)
    else:
        run_ours(args, L, rank, world, local_rank)


if __name__ == "__main__":
    main()
