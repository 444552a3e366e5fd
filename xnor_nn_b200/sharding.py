"""Minibatch slicing for multi-GPU runs.

Every stage of the path is independent per image (the minibatch is upstream's outermost loop
everywhere, e.g. src/default/bcast_convolution_default.cpp:61), and NCHW/NHWC tensors are
contiguous per image, so rank r of N owns a contiguous run of images and nothing is exchanged:
the packed weights are derived locally from the fp32 weights every rank holds.
"""


def shard_range(mb, rank, world):
    """[first, last) images of `rank`; sizes differ by at most one when world does not divide mb."""
    if not (0 <= rank < world) or mb < 0:
        raise ValueError("bad shard request")
    return mb * rank // world, mb * (rank + 1) // world


def shard_sizes(mb, world):
    return [shard_range(mb, r, world)[1] - shard_range(mb, r, world)[0] for r in range(world)]
