"""Times AlexNet's conv3 -> conv4 -> conv5 (13x13, 3x3, pad 1: 256 -> 384 -> 256 -> 256 channels)
layer by layer and as one chained call, tensors resident on the device.

    python -m xnor_nn_b200.chain_case [MINIBATCH=256] [REPS=60]

Prints one JSON line with microseconds per pass (CUDA events on the launching stream, six rotating
tensor sets so that a pass does not find its inputs in L2).
"""
import json
import sys

import xnor_nn_b200 as xb
from xnor_nn_b200 import synth

CHANNELS = (256, 384, 256, 256)


def main(argv):
    import torch
    mb = int(argv[1]) if len(argv) > 1 else 256
    reps = int(argv[2]) if len(argv) > 2 else 60
    convs = []
    for i in range(3):
        ic, oc = CHANNELS[i], CHANNELS[i + 1]
        w = synth.normal(0xBEEF0000 + i, oc * ic * 9, 0.05)
        convs.append(xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, mb, oc, ic, 13,
                                    13, 3, 3, 1, 1, 1, 1, w))
    stream = torch.cuda.current_stream().cuda_stream
    for cv in convs:
        cv.set_stream(stream)
    sets = 6
    bufs = [[torch.randn(mb * c * 169, device="cuda") for c in CHANNELS] for _ in range(sets)]

    def timed(fn):
        for i in range(30):  # warm-up: clocks and caches settle
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

    out = {"minibatch": mb, "reps": reps, "unit": "us per pass",
           "conv3_conv4": {"layer_by_layer": timed(separate(2)), "chained": timed(chained(2))},
           "conv3_conv4_conv5": {"layer_by_layer": timed(separate(3)), "chained": timed(chained(3))}}
    print(json.dumps(out))
    for cv in convs:
        cv.close()


if __name__ == "__main__":
    main(sys.argv)
