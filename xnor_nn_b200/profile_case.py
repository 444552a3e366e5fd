"""Small driver for profilers: a few forward passes of one benchmark layer, tensors on the device.

    python -m xnor_nn_b200.profile_case [CONFIG=B] [MINIBATCH] [PASSES=3] [KERNEL=auto]

Meant to be wrapped by `ncu` on a reduced minibatch so that a capture of a handful of launches
ends by itself (a few hundred MB on the device, one weight set-up and PASSES x 2 kernels).
"""
import sys

import numpy as np

import xnor_nn_b200 as xb
from xnor_nn_b200 import synth


def main(argv):
    import torch
    cfg = argv[1] if len(argv) > 1 else "B"
    L = synth.CONFIGS[cfg]
    mb = int(argv[2]) if len(argv) > 2 else L.mb
    passes = int(argv[3]) if len(argv) > 3 else 3
    kernel = {"auto": xb.KERNEL_AUTO, "popc": xb.KERNEL_POPC,
              "tcgen05_i8": xb.KERNEL_TCGEN05_I8}[argv[4] if len(argv) > 4 else "auto"]
    src, w = synth.make_inputs(cfg, mb=mb)
    conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, mb, L.oc, L.ic, L.ih,
                          L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w, kernel=kernel)
    d_src = torch.from_numpy(src).cuda()
    d_dst = torch.empty(int(np.prod(conv.out_shape)), device="cuda")
    for _ in range(passes):
        conv.forward(d_src, d_dst)
    conv.synchronize()
    print("ok", xb.KERNEL_NAMES[conv.kernel], "mb=%d passes=%d" % (mb, passes))
    conv.close()


if __name__ == "__main__":
    main(sys.argv)
