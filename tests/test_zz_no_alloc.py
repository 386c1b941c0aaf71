"""strix_b200_gemv_noalloc against strix_gemv, through the C ABI.

The entry point serves callers that cannot give the GEMV any scratch memory (an engine
whose arena owns all device memory, so that neither a workspace nor a cudaMalloc is
available inside its decode loop).  Its scratch is a fixed array inside the library, shared
by every call; a call marks the planes it is going to use empty before its kernel starts, so
the test runs it twice in a row on different inputs: whatever the first call left in the
array must not leak into the second.  (The array is sized for eight rows on up to 256 SMs, so
no layer is beyond it on a B200: the refusal of a larger launch cannot be provoked here.)  The
file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from strix_trellis_b200 import native as N, synthetic
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def test_noalloc_matches_workspace_gemv_twice_in_a_row():
    from strix_trellis_b200.runtime import Context
    ctx = Context(0)
    lib = N.load()
    sd = N.stream_desc(torch.cuda.current_stream().cuda_stream)
    cases = [(4096, 4096, 4, 1, 31), (1152, 4096, 5, 8, 32), (4096, 4096, 4, 3, 33)]
    for inputs, outputs, bits, rows, seed in cases:
        layer = synthetic.make_layer(inputs, outputs, bits, seed=seed, bias=True)
        w = ctx.prepare(layer)
        for call in range(2):  # two calls in a row share the built-in scratch
            x = dev(synthetic.make_activations(rows, inputs, seed=seed * 10 + call))
            want = w.gemv(x)                      # existing entry point, caller workspace
            got = torch.full((rows, outputs), float("nan"), device="cuda")
            d = w.matmul_desc(x, got)             # workspace stays NULL/0
            N.check(lib.strix_b200_gemv_noalloc(ctx.handle, C.byref(d), C.byref(sd)), "strix_b200_gemv_noalloc")
            torch.cuda.synchronize()
            # same kernel, same partition, same fold order: the results are bit-identical
            assert host(got).tobytes() == host(want).tobytes(), (inputs, outputs, bits, rows, call)
        # alpha/beta through the same path
        old = torch.randn((rows, outputs), device="cuda")
        y1, y2 = old.clone(), old.clone()
        w.gemv(x, y1, alpha=-0.5, beta=0.25)
        d = w.matmul_desc(x, y2, alpha=-0.5, beta=0.25)
        N.check(lib.strix_b200_gemv_noalloc(ctx.handle, C.byref(d), C.byref(sd)), "strix_b200_gemv_noalloc")
        torch.cuda.synchronize()
        assert host(y1).tobytes() == host(y2).tobytes()
        # a workspace is refused: the point of the call is that none exists
        ws = torch.empty(4096, dtype=torch.uint8, device="cuda")
        d = w.matmul_desc(x, y2, workspace=ws)
        assert lib.strix_b200_gemv_noalloc(ctx.handle, C.byref(d), C.byref(sd)) == N.INVALID_ARGUMENT
        w.close()
    assert ctx.device_status() == 0
    ctx.close()
