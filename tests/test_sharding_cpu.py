"""The multi-GPU path on CPU: two gloo ranks each take their minibatch slice, run the (CPU
oracle) forward on it, and the gathered result equals the unsharded forward. Covers the slicing
arithmetic, the per-image input generation that lets ranks build their slices independently, and
the max-over-ranks reduction the benchmark uses for timing."""
import os
import socket
import sys

import numpy as np
import pytest

from xnor_nn_b200 import sharding, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_tile_the_minibatch():
    for mb in (1, 7, 64, 256):
        for world in (1, 2, 3, 4, 8):
            edges = [sharding.shard_range(mb, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == mb
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
            sizes = sharding.shard_sizes(mb, world)
            assert sum(sizes) == mb and max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def test_slices_of_the_synthetic_batch_are_position_independent():
    full, w = synth.make_inputs("A", mb=6)
    part, w2 = synth.make_inputs("A", mb=2, first_image=3)
    assert np.array_equal(full[3:5], part) and np.array_equal(w, w2)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle.pyoracle import Oracle, Shape
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L = synth.layer_shape("A", mb=5)  # 5 images on 2 ranks: slices of 2 and 3
        first, last = sharding.shard_range(L.mb, rank, world)
        src, w = synth.make_inputs("A", mb=last - first, first_image=first)
        s = Shape.make(last - first, L.oc, L.ic, L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw)
        mine = Oracle().convolution(s, src, w)["dst"]
        # host gather, as the benchmark's ranks would hand their slices back
        parts = [None] * world
        dist.all_gather_object(parts, (first, mine))
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # the timing reduction
        if rank == 0:
            parts.sort(key=lambda p: p[0])
            np.save(out, np.concatenate([p[1] for p in parts]))
            assert t.item() == world
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_forward(tmp_path, oracle):
    import torch.multiprocessing as mp
    from oracle.pyoracle import Shape
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    out = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    L = synth.layer_shape("A", mb=5)
    src, w = synth.make_inputs("A", mb=5)
    s = Shape.make(L.mb, L.oc, L.ic, L.ih, L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw)
    assert np.array_equal(np.load(out), oracle.convolution(s, src, w)["dst"])
