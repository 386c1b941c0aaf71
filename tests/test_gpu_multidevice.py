"""Two contexts on two devices in ONE process: kernel attributes (the opt-in shared-memory size
of every instantiation) are per device, so a context created on a second device must be set up
on its own -- every route that needs the opt-in size fails to launch there otherwise.  Needs two
visible GPUs; the CPU contract test covers the same rule against a fake runtime."""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from strix_trellis_b200 import synthetic
from gpu_util import gate

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_in_the_same_process():
    from strix_trellis_b200.runtime import Context
    layer = synthetic.make_layer(2048, 1024, 4, 9700, bias=True)
    x1 = synthetic.make_activations(1, 2048, seed=9701)   # one-row kernel
    x8 = synthetic.make_activations(8, 2048, seed=9702)   # multi-row kernel
    xm = synthetic.make_activations(600, 2048, seed=9703)  # tensor-core pair kernel
    want = {k: c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, 4, 2, v)
            for k, v in (("r1", x1), ("r8", x8), ("m", xm))}
    got = {}
    contexts = []
    for device in (0, 1):  # device 0 first: its set-up must not stand in for device 1's
        with torch.cuda.device(device):
            ctx = Context(device)
            contexts.append(ctx)
            w = ctx.prepare(layer)
            put = lambda a: torch.from_numpy(a).cuda(device)
            got[device] = {"r1": w.gemv(put(x1)).cpu().numpy(), "r8": w.gemv(put(x8)).cpu().numpy(),
                           "m": w.gemm(put(xm)).cpu().numpy()}
            torch.cuda.synchronize(device)
            assert ctx.device_status() == 0
            w.close()
    for device in (0, 1):
        for k in want:
            gate(got[device][k], want[k], f"device {device} {k}")
    for k in want:  # same kernels, same inputs: same bits on both devices
        assert got[0][k].tobytes() == got[1][k].tobytes(), k
    for device, ctx in enumerate(contexts):
        with torch.cuda.device(device):
            ctx.close()
