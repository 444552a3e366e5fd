"""A bounded device wait that runs out, in the form that leaves the GPU healthy: the library's
test hook shortens the kernels' wait limit to a few milliseconds and makes one thread block skip
the tcgen05.commit that publishes its first result tile. Nothing faults, traps or spins without a
bound: the warps waiting for that tile give up when the limit expires, every role of every block
winds down, the kernel returns, and the host turns the recorded error word into a status."""
import ctypes as C

import numpy as np
import pytest

import xnor_nn_b200 as xb
from xnor_nn_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kernel", [xb.KERNEL_TCGEN05_I8, xb.KERNEL_TCGEN05_I8_ROWS],
                         ids=["tcgen05_i8", "tcgen05_i8_rows"])
# one image; 40 images: one tile per thread block on many SMs; 256 images: several tiles per block,
# the position-tile kernel on CTA pairs (the block that loses its commit is a pair's leader, so
# both blocks of the pair give up, keep the epilogue's meetings and leave through the cluster
# barrier)
@pytest.mark.parametrize("mb", [1, 40, 256])
def test_lost_commit_times_out_and_the_resources_stay_usable(kernel, mb):
    torch = pytest.importorskip("torch")
    L = synth.layer_shape("A", mb=mb)
    src, w = synth.make_inputs("A", mb=mb)
    conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, L.mb, L.oc, L.ic, L.ih,
                          L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w, kernel=kernel)
    assert conv.kernel == kernel
    d_src = torch.from_numpy(src).cuda()
    good = torch.zeros(int(np.prod(conv.out_shape)), device="cuda")
    conv.forward(d_src, good)
    conv.synchronize()

    junk = torch.zeros_like(good)
    conv._set(xb.SLOT_USER_DST, junk)
    st = xb.lib().xnor_nn_b200_selftest_lost_commit(C.byref(conv.c), conv.res, 5)
    assert st == xb.UNIMPLEMENTED
    # The first wait to run out names the site. With one tile per block that is an epilogue warp
    # waiting for the lost tile (4). With several tiles the waits that depend on that tile start
    # within microseconds of one another (the MMA issuers waiting for its accumulator to be handed
    # back, 2 and 6, the producer behind them, 1 and 8): whichever expires first is recorded.
    err = xb.last_error()
    if mb == 256:
        assert "gave up waiting (site " in err, err
    else:
        assert "gave up waiting (site 4)" in err, err
    # the error word was consumed: the next synchronising call is clean again
    conv.synchronize()

    again = torch.zeros_like(good)
    conv.forward(d_src, again)
    conv.synchronize()
    assert torch.equal(again, good)
    conv.close()


def test_hook_refuses_what_it_cannot_run():
    L = synth.layer_shape("A", mb=1)
    _, w = synth.make_inputs("A", mb=1)
    conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, L.mb, L.oc, L.ic, L.ih,
                          L.iw, L.kh, L.kw, L.sh, L.sw, L.ph, L.pw, w, kernel=xb.KERNEL_POPC)
    host = np.zeros(int(np.prod(conv.out_shape)), np.float32)
    conv._set(xb.SLOT_USER_DST, host)
    st = xb.lib().xnor_nn_b200_selftest_lost_commit(C.byref(conv.c), conv.res, 5)
    assert st == xb.ERROR_INVALID_INPUT
    conv.close()
