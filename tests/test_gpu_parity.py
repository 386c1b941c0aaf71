"""GPU parity tests: every call goes through the C ABI of libstrix_trellis.so."""
import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import c_oracle, trellis_ref as ref
from strix_trellis_b200 import native as N, synthetic
from gpu_util import dev, gate, host

pytestmark = pytest.mark.gpu


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def ctx():
    from strix_trellis_b200.runtime import Context
    c = Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


@pytest.fixture(scope="module")
def grid(golden_dir):
    meta = json.loads((golden_dir / "grid.json").read_text())
    return meta, np.load(golden_dir / "grid_ref.npz")


def test_stage_probes_bit_exact_on_reference_grid(ctx, grid):
    """Decoded Q, scaled fp16, input H128, core input, exact-order core and the output
    stages must equal the reference's checkpoints bit for bit (all 48 grid cases)."""
    meta, outs = grid
    for case in meta["cases"]:
        layer, x, old, _ = synthetic.grid_case(case["codebook"], case["bits"], case["wide"], meta["rows"])
        for use_blob in (False, True):
            w = ctx.prepare(layer, use_blob=use_blob)
            assert sha(host(w.dequantize())) == case["q"], case["name"]
            if use_blob:
                w.close()
                continue
            scaled, had, core_in = w.input_stages(dev(x))
            assert sha(host(scaled)) == case["scaled"], case["name"]
            assert sha(host(had)) == case["inh"], case["name"]
            assert sha(host(core_in)) == case["a"], case["name"]
            core = w.core_exact(core_in)
            assert sha(host(core)) == case["core"], case["name"]
            y = w.output_stages(core)
            assert sha(host(y)) == case["ref"], case["name"]
            # output stages on the oracle's core, with alpha/beta and an old output
            for alpha, beta in [(-0.75, 0.25), (0.0, -0.5), (1.0, -0.0)]:
                yy = dev(old.copy())
                w.output_stages(dev(outs[case["name"] + ":core"]), alpha, beta, yy)
                want = c_oracle.output_stages(outs[case["name"] + ":core"], layer.svh, layer.bias, alpha, beta, old)["output"]
                assert host(yy).tobytes() == want.tobytes(), (case["name"], alpha, beta)
            w.close()


def test_output_stage_folds_split_planes_in_order(ctx):
    layer = synthetic.make_layer(128, 256, 4, seed=11, bias=True)
    w = ctx.prepare(layer)
    rng = np.random.default_rng(3)
    planes = (rng.normal(size=(5, 3, 256)) * 10.0 ** rng.integers(-3, 4, (5, 3, 256))).astype(np.float32)
    acc = np.zeros((3, 256), np.float32)
    for s in range(5):
        acc = acc + planes[s]
    want = c_oracle.output_stages(acc, layer.svh, layer.bias)["output"]
    assert host(w.output_stages(dev(planes))).tobytes() == want.tobytes()
    w.close()


@pytest.mark.parametrize("rows", [1, 2, 3, 8])
def test_gemv_grid_all_rates_and_codebooks(ctx, grid, rows):
    meta, outs = grid
    for case in meta["cases"]:
        layer, x, old, _ = synthetic.grid_case(case["codebook"], case["bits"], case["wide"], meta["rows"])
        w = ctx.prepare(layer)
        y = w.gemv(dev(x[:rows]))
        gate(host(y), outs[case["name"]][:rows], case["name"])
        w.close()


def test_gemv_rank1_alpha_beta_and_poisoned_output(ctx, grid):
    meta, outs = grid
    for case in meta["cases"][::5]:
        layer, x, old, _ = synthetic.grid_case(case["codebook"], case["bits"], case["wide"], meta["rows"])
        w = ctx.prepare(layer)
        want = outs[case["name"]]
        y1 = w.gemv(dev(x[0]))
        assert y1.shape == (layer.outputs,)
        gate(host(y1)[None], want[:1], case["name"])
        for alpha, beta in [(-0.75, 0.25), (0.0, -0.5)]:
            y = dev(old[:4].copy())
            w.gemv(dev(x[:4]), y, alpha, beta)
            gate(host(y), ref.apply_alpha_beta(want[:4], alpha, beta, old[:4]), case["name"])
        for beta in (0.0, -0.0):  # beta == 0 must never read the old output
            y = torch.full((4, layer.outputs), float("nan"), device="cuda")
            w.gemv(dev(x[:4]), y, 1.0, beta)
            gate(host(y), want[:4], case["name"])
        w.close()


def test_gemv_non_finite_inputs_fold_without_waiting(ctx):
    """The split-K fold tells a published word from an unwritten one by its bit pattern (an
    all-ones NaN).  NaN and infinite activations must come out as ordinary NaN/inf results:
    no wait may run out (status word stays 0), other rows are unaffected, and the scratch is
    left reusable (the same plan is submitted again with finite inputs)."""
    layer = synthetic.make_layer(4096, 512, 4, seed=61, bias=True)  # 4 column blocks: every block is split
    w = ctx.prepare(layer)
    x = synthetic.make_activations(3, 4096, seed=62)
    bad = x.copy()
    bad[0, 5] = np.nan
    bad[1, 700] = np.inf
    bad[1, 701] = -np.inf
    xd, y = dev(bad), torch.zeros((3, 512), device="cuda")
    ws = torch.empty(max(w.workspace_bytes(xd, y), 256), dtype=torch.uint8, device="cuda")
    plan = w.plan(xd, y, N.OP_GEMV, workspace=ws)
    plan.submit()
    torch.cuda.synchronize()
    got = host(y)
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, 4, 2, x)
    assert ctx.device_status() == 0
    assert np.isnan(got[0]).all() and not np.isfinite(got[1]).any()
    gate(got[2:], want[2:], "finite row beside non-finite rows")
    xd.copy_(dev(x))
    plan.submit()
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    gate(host(y), want, "same scratch after non-finite inputs")
    plan.close()
    w.close()


def test_empty_call_validates_and_launches_nothing(ctx):
    layer = synthetic.make_layer(128, 128, 4, seed=5)
    w = ctx.prepare(layer)
    x = torch.empty((0, 128), device="cuda")
    y = torch.empty((0, 128), device="cuda")
    assert w.workspace_bytes(x, y) == 0
    w.gemv(x, y)
    w.gemm(x, y)
    w.close()


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6])
@pytest.mark.parametrize("shape", [(4096, 4096), (5120, 5120), (1152, 4096), (4096, 14336)])
def test_gemv_benchmark_shapes(ctx, bits, shape):
    inputs, outputs = shape
    layer = synthetic.make_layer(inputs, outputs, bits, seed=synthetic.BASE_SEED + bits)
    w = ctx.prepare(layer)
    x = synthetic.make_activations(8, inputs, seed=synthetic.BASE_SEED + 100 + bits)
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, bits, 2, x)
    for rows in (1, 2, 4, 8):
        gate(host(w.gemv(dev(x[:rows]))), want[:rows], f"k{bits} {shape} r{rows}")
    w.close()


@pytest.mark.parametrize("shape", [(128, 128), (256, 128), (16384, 128), (8192, 256), (128, 4096), (384, 19072),
                                   (1152, 4096), (32768, 256), (33024, 128)])
def test_gemv_one_row_fold_shapes(ctx, shape):
    """One activation row through every way a column block can be finished: one CTA alone
    (128x128), a block shared by more CTAs than there are decode warps (16384 -> 128: 127
    planes gathered in rounds of sixteen), blocks that lie wholly inside a CTA's range next to
    shared ones (384 -> 19072), the widest row the one-row kernel stages at once (32768) and one
    block more (33024: falls back to the staged-per-segment kernel).  Each layer is submitted
    three times on ONE plan and scratch area: the planes must come back empty every time and
    the bits must not depend on arrival order."""
    inputs, outputs = shape
    bits = 2 + (inputs // 128 + outputs // 128) % 5
    layer = synthetic.make_layer(inputs, outputs, bits, seed=4000 + inputs // 128, bias=bool(outputs % 256))
    w = ctx.prepare(layer)
    x = synthetic.make_activations(1, inputs, seed=4001)
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, bits, 2, x)
    xd, y = dev(x), torch.zeros((1, outputs), device="cuda")
    plan = w.plan(xd, y, N.OP_GEMV)
    seen = None
    for turn in range(3):
        y.fill_(float("nan"))
        plan.submit()
        torch.cuda.synchronize()
        assert ctx.device_status() == 0
        gate(host(y), want, f"{shape} K{bits} submit {turn}")
        seen = host(y).tobytes() if seen is None else seen
        assert host(y).tobytes() == seen
    # rank-1 call with alpha / beta over a poisoned and over a real old output
    old = synthetic.rng_for(4002).normal(0, 0.3, (1, outputs)).astype(np.float32)
    yy = dev(old.copy())
    w.gemv(xd, yy, alpha=-0.75, beta=0.25)
    gate(host(yy), ref.apply_alpha_beta(want, -0.75, 0.25, old), f"{shape} alpha/beta")
    plan.close()
    w.close()


@pytest.mark.parametrize("shape,rows", [((4096, 129280), 1), ((16384, 4096), 8)])
def test_gemv_tensor_parallel_layer_shapes(ctx, shape, rows):
    """The two dense layers of the tensor-parallel benchmark configuration, unsharded, K5:
    the LM head (1010 column blocks, 218 units per CTA) and the 16384-input projection
    (128 H128 blocks: at 8 rows the core input exceeds the staging area and is staged per
    segment)."""
    layer = synthetic.make_layer(shape[0], shape[1], 5, seed=300 + rows)
    x = synthetic.make_activations(rows, shape[0], seed=301)
    w = ctx.prepare(layer)
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, 5, 2, x)
    gate(host(w.gemv(dev(x))), want, f"K5 {shape} rows {rows}")
    assert ctx.device_status() == 0
    w.close()


def test_half_integer_rates_decode_bit_exact_and_multiply(ctx, golden_dir):
    """Rates 1.5 / 2.5 / 3.5 (stream positions alternate between floor(rate) and one bit more,
    mul1 only; reference python/strix_trellis/codec.py:12-20, CPU-only there).  The decoded Q of
    the golden tiles carries the hash the reference's own decoder produced; a larger layer goes
    through the one-row kernel, the multi-row kernel, the 8-row chunks and the tensor-core GEMM
    against the NumPy contract."""
    meta = json.loads((golden_dir / "half_rates.json").read_text())
    rng = synthetic.rng_for(synthetic.BASE_SEED + 50)
    ones, more_ones = np.ones(128, np.float16), np.ones(128, np.float16)  # two regions may not share bytes
    for rate in (1.5, 2.5, 3.5):
        t = rng.integers(0, 65536, (8, 8, int(16 * rate)), dtype=np.uint16)
        w = ctx.prepare(synthetic.Layer(t, ones, more_ones, None, rate, "mul1"))
        assert sha(host(w.dequantize())) == meta[str(rate)]["q"]
        w.close()
        layer = synthetic.make_layer(512, 384, rate, seed=7000 + int(rate * 2), bias=True)
        x = synthetic.make_activations(100, 512, seed=7001)
        want = ref.linear_stages(x, layer.trellis, layer.suh, layer.svh, rate, "mul1", layer.bias)["output_fp32"]
        w = ctx.prepare(layer)
        assert host(w.dequantize()).tobytes() == ref.dequantize(layer.trellis, rate, "mul1").tobytes()
        for rows in (1, 3, 8):
            gate(host(w.gemv(dev(x[:rows]))), want[:rows], f"rate {rate} gemv rows {rows}")
        for rows in (12, 20, 100):
            gate(host(w.gemm(dev(x[:rows]))), want[:rows], f"rate {rate} gemm rows {rows}")
        _, _, core_in = w.input_stages(dev(x[:2]))
        exact = w.output_stages(w.core_exact(core_in))
        assert host(exact).tobytes() == want[:2].tobytes()  # reference accumulation order: identical bits
        assert ctx.device_status() == 0
        w.close()
    with pytest.raises((ValueError, N.StrixError)):  # half-integer rates exist for mul1 only
        ctx.prepare(synthetic.Layer(t, ones, more_ones, None, 3.5, "mcg"))


@pytest.mark.parametrize("rows", [1, 5, 12, 24, 300])
def test_half_precision_tensors_widen_on_load_and_round_on_store(ctx, rows):
    """binary16 / bfloat16 activations and outputs (reserved and refused by the reference,
    include/strix_trellis.h:39-40; honoured here).  The arithmetic is the float32 contract: an
    input of either type gives the bits of the same values passed as float32, and an output of
    either type is the float32 output rounded to nearest even -- through the one-row kernel, the
    multi-row kernel, the 8-row chunks and the tensor-core GEMM, with and without alpha / beta
    over an old output of that type."""
    layer = synthetic.make_layer(1024, 640, 4, seed=8100 + rows, bias=True)
    w = ctx.prepare(layer)
    run = w.gemv if rows <= 8 else w.gemm
    x32 = synthetic.make_activations(rows, 1024, seed=8101)  # binary16-representable values
    want32 = host(run(dev(x32)))
    gate(want32, c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, 4, 2, x32), "float32 tensors")
    for dtype in (torch.float16, torch.bfloat16):
        xin = dev(x32).to(dtype)                       # bfloat16 drops bits: compare against the widened values
        base = run(xin.to(torch.float32))
        y32 = run(xin)
        assert torch.equal(y32, base), dtype           # widening on load is exact
        y = torch.empty((rows, 640), dtype=dtype, device="cuda")
        run(xin, y)
        assert torch.equal(y, base.to(dtype)), dtype   # one rounding, to nearest even
        old = (torch.randn((rows, 640), device="cuda") * 0.25).to(dtype)
        y2 = old.clone()
        run(xin, y2, alpha=-0.75, beta=0.5)
        expect = (base * -0.75 + old.to(torch.float32) * 0.5).to(dtype)  # each product rounded, then the sum, then the store
        assert torch.equal(y2, expect), dtype
    # a strided float16 row view through a tensor-parallel dense plan
    if rows <= 8:
        from strix_trellis_b200.runtime import DensePlan
        wide = torch.zeros((rows, 1536), dtype=torch.float16, device="cuda")
        wide[:, 256:1280] = dev(x32).to(torch.float16)
        out = torch.zeros((rows, 1024), dtype=torch.bfloat16, device="cuda")
        plan = DensePlan(w, wide[:, 256:1280], out[:, 128:768])
        plan.submit()
        torch.cuda.synchronize()
        assert torch.equal(out[:, 128:768], torch.from_numpy(want32).cuda().to(torch.bfloat16))
        assert float(out[:, :128].abs().max()) == 0.0 and float(out[:, 768:].abs().max()) == 0.0
        plan.close()
    assert ctx.device_status() == 0
    w.close()


def test_config1_against_reference_golden(ctx, golden_dir):
    meta = json.loads((golden_dir / "config1.json").read_text())
    gold = np.load(golden_dir / "config1.npz")
    layer = synthetic.make_layer(4096, 4096, 4, seed=meta["seed"])
    x = synthetic.make_activations(1, 4096, seed=meta["x_seed"])
    w = ctx.prepare(layer)
    assert sha(host(w.dequantize())) == meta["q"]
    _, _, core_in = w.input_stages(dev(x))
    assert sha(host(core_in)) == meta["a"]
    core = w.core_exact(core_in)
    assert sha(host(core)) == meta["core"]           # reference accumulation order reproduced
    assert sha(host(w.output_stages(core))) == meta["ref"]
    gate(host(w.gemv(dev(x))), gold["ref"], "config1 fused")
    w.close()


@pytest.mark.parametrize("rows", [9, 16, 17, 32])
def test_gemm_small_rows(ctx, grid, rows):
    """Up to 16 rows run as 8-row chunks of the fused GEMV, more rows take the tcgen05 kernel."""
    meta, outs = grid
    for case in meta["cases"][::7]:
        layer, _, _, _ = synthetic.grid_case(case["codebook"], case["bits"], case["wide"], meta["rows"])
        x = synthetic.make_activations(rows, layer.inputs, seed=77)
        w = ctx.prepare(layer)
        want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, layer.bits, case["codebook"], x)
        gate(host(w.gemm(dev(x))), want, case["name"])
        w.close()


@pytest.mark.parametrize("rows", [40, 64, 128, 200, 256, 300, 513, 1030])
def test_gemm_tensor_core_small_layers(ctx, grid, rows):
    """More than 16 rows take the tcgen05 kernels: every rate and codebook, ragged row counts."""
    meta, outs = grid
    for case in meta["cases"][::3]:
        layer, _, _, _ = synthetic.grid_case(case["codebook"], case["bits"], case["wide"], meta["rows"])
        x = synthetic.make_activations(rows, layer.inputs, seed=78)
        old = synthetic.rng_for(79).normal(0, 0.3, (rows, layer.outputs)).astype(np.float32)
        w = ctx.prepare(layer)
        want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, layer.bits, case["codebook"], x)
        gate(host(w.gemm(dev(x))), want, case["name"])
        y = dev(old.copy())
        w.gemm(dev(x), y, alpha=-0.75, beta=0.25)
        gate(host(y), ref.apply_alpha_beta(want, -0.75, 0.25, old), case["name"] + " alpha/beta")
        w.close()


@pytest.mark.parametrize("rows", [100, 256, 512])
@pytest.mark.parametrize("bits", [4, 5, 6])
def test_gemm_tensor_core_prefill_shape(ctx, bits, rows):
    """4096 -> 1536 slice of the benchmark's fused-QKV-like layer.  Up to 256 rows there is one
    row tile and K is partitioned over the idle SMs (raw partial accumulators, folded in
    ascending K order by a finishing kernel); 512 rows take the unpartitioned route."""
    layer = synthetic.make_layer(4096, 1536, bits, seed=90 + bits, bias=True)
    x = synthetic.make_activations(rows, 4096, seed=91)
    old = synthetic.rng_for(92).normal(0, 0.3, (rows, 1536)).astype(np.float32)
    w = ctx.prepare(layer)
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, bits, 2, x)
    gate(host(w.gemm(dev(x))), want, f"prefill k{bits} rows {rows}")
    y = dev(old.copy())
    w.gemm(dev(x), y, alpha=0.5, beta=-1.0)
    gate(host(y), ref.apply_alpha_beta(want, 0.5, -1.0, old), f"prefill k{bits} rows {rows} alpha/beta")
    w.close()


@pytest.mark.parametrize("rows", [40, 130, 300])
def test_gemm_more_column_stripes_than_sms(ctx, rows):
    """A wide, short layer (256 -> 40960: 160 column stripes of 256, four K steps each): with up
    to 256 rows some CTAs of the single-CTA kernel run two work items, so the weight prefetch and
    the decoders' look-ahead cross from one item into the next and only the last item's
    epilogue is shared with the decoder warps; 300 rows take the two-CTA kernel the same way."""
    layer = synthetic.make_layer(256, 40960, 2, seed=640, bias=True)
    x = synthetic.make_activations(rows, 256, seed=641)
    w = ctx.prepare(layer)
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, 2, 2, x)
    gate(host(w.gemm(dev(x))), want, f"wide layer rows {rows}")
    assert ctx.device_status() == 0
    w.close()


@pytest.mark.parametrize("bits,rows", [(4, 8192), (4, 2048), (5, 2048), (5, 8192), (6, 2048), (6, 8192)])
def test_gemm_full_prefill_size_sampled_rows_and_linearity(ctx, bits, rows):
    """The benchmark's prefill layer at full width (4096 -> 12288) in one launch, at every rate
    and at both large row counts it is timed on.  The CPU contract is evaluated on a sample of
    rows spread over all row tiles (every 331st row and the last one); the whole output is
    checked through properties that need no reference: the fused GEMV of the same rows agrees
    within the gates, and alpha/beta act linearly (the reference streams its large heads through
    column blocks and gates them globally and per row the same way,
    tools/make_full_head_cpu_reference.py:29-45,86-105)."""
    layer = synthetic.make_layer(4096, 12288, bits, seed=500 + bits, bias=True)
    x = synthetic.make_activations(rows, 4096, seed=501 + rows)
    w = ctx.prepare(layer)
    xd = dev(x)
    y = w.gemm(xd)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    sample = sorted(set(list(range(0, rows, 331)) + [rows - 1]))
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, bits, 2, np.ascontiguousarray(x[sample]))
    got = host(y[sample])
    gate(got, want, f"K{bits} {rows}-row prefill, sampled rows")
    assert bool(torch.isfinite(y).all())
    # the GEMV route on eight of the sampled rows: another kernel, same contract
    pick = sample[:8]
    gate(host(w.gemv(dev(np.ascontiguousarray(x[pick])))), want[:8], "gemv on sampled rows")
    # y2 = -0.5 * Linear(x) + 2 * y  ==  1.5 * y, elementwise within float32 rounding of the two products
    y2 = y.clone()
    w.gemm(xd, y2, alpha=-0.5, beta=2.0)
    torch.cuda.synchronize()
    expect = host(y) * np.float32(1.5)
    np.testing.assert_allclose(host(y2), expect, rtol=2e-6, atol=1e-6 * float(np.abs(expect).max()))
    w.close()


def test_plan_submit_and_graph_replay(ctx):
    layer = synthetic.make_layer(4096, 1024, 5, seed=21, bias=True)
    w = ctx.prepare(layer)
    x = dev(synthetic.make_activations(4, 4096, seed=22))
    y = torch.zeros((4, 1024), device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        plan = w.plan(x, y, N.OP_GEMV, stream=stream)
        plan.submit()
        stream.synchronize()
        want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, 5, 2, host(x))
        gate(host(y), want, "plan")
        first = host(y).copy()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            plan.submit()
        for trial in range(3):
            x2 = synthetic.make_activations(4, 4096, seed=30 + trial)
            x.copy_(dev(x2))
            y.fill_(float("nan"))
            graph.replay()
            stream.synchronize()
            gate(host(y), c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, 5, 2, x2), "graph")
        # same inputs -> same bits, run to run
        x.copy_(dev(synthetic.make_activations(4, 4096, seed=22)))
        plan.submit()
        stream.synchronize()
        assert host(y).tobytes() == first.tobytes()
        del graph
        assert N.load().strix_weights_destroy(w.handle) == N.INVALID_ARGUMENT  # retained by the plan
        plan.close()
    w.close()


def test_rejections_with_the_real_driver(ctx):
    """Host memory, short and misaligned workspace, aliasing: rejected before any launch
    (the reference's real-driver negative cases, tests/gpu_runtime.hip:189-219)."""
    import ctypes as C
    # K so deep that the split-K fold needs global scratch (more partitions than a cluster holds)
    layer = synthetic.make_layer(34816 * 2, 128, 2, seed=9)
    w = ctx.prepare(layer)
    lib = N.load()
    x = dev(synthetic.make_activations(8, 34816 * 2))
    y = torch.full((8, 128), 7.0, device="cuda")
    need = w.workspace_bytes(x, y)
    assert need > 0
    ws = torch.empty(need + 512, dtype=torch.uint8, device="cuda")
    sd = N.stream_desc(torch.cuda.current_stream().cuda_stream)

    def status(d):
        return lib.strix_gemv(ctx.handle, C.byref(d), C.byref(sd))

    d = w.matmul_desc(x, y, workspace=ws[: need - 256])
    assert status(d) == N.INSUFFICIENT_BUFFER
    d = w.matmul_desc(x, y, workspace=ws[4: need + 4])
    assert status(d) == N.INVALID_ARGUMENT
    d = w.matmul_desc(x, x[:, :128], workspace=ws)
    assert status(d) in (N.INVALID_ARGUMENT, N.UNSUPPORTED_FORMAT)
    hx = torch.zeros((8, 34816 * 2)).pin_memory()
    d = w.matmul_desc(x, y, workspace=ws)
    d.input.data = hx.data_ptr()
    assert status(d) == N.INVALID_ARGUMENT
    d = w.matmul_desc(x, y, workspace=ws)
    d.alpha = float("inf")
    assert status(d) == N.INVALID_ARGUMENT
    d = w.matmul_desc(x, y, workspace=ws)
    for bad_dtype in (0, 7):  # 1, 2, 3 are binary16, bfloat16, float32
        d.input.dtype = bad_dtype
        assert status(d) == N.UNSUPPORTED_FORMAT
    torch.cuda.synchronize()
    assert (host(y) == 7.0).all()  # nothing ran
    # and the deep-K global-scratch path itself is correct
    got = w.gemv(x, workspace=ws)
    want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, 2, 2, host(x))
    gate(host(got), want, "deep K global fold")
    w.close()


def test_decode_rate_probe_reports_a_plausible_cost(ctx):
    """The decoder-only probe: a positive, finite number of SM clocks per tile for every rate and
    warp count it accepts (the decoder of any rate needs more than 20 and far fewer than 400
    clocks), and a refusal for warp counts that do not fill the SM's four sub-partitions evenly."""
    for bits in (2, 4, 5):
        w = ctx.prepare(synthetic.make_layer(256, 256, bits, 4400 + bits))
        for warps in (8, 16, 32):
            clocks = w.decode_rate(20, warps_per_sm=warps)
            assert 20.0 < clocks < 400.0, (bits, warps, clocks)
        for bad in (0, 2, 18, 36):
            with pytest.raises(N.StrixError):
                w.decode_rate(20, warps_per_sm=bad)
        w.close()
    assert ctx.device_status() == 0
