"""The frozen-plan family of the C ABI on the GPU: per-rank dense plans on strided row views,
paired projections, the SwiGLU plan, the grouped strided GEMV and the pre-routed grouped call,
each against the CPU contract of the same linears."""
import ctypes as C
import numpy as np
import pytest
import torch

from oracle import c_oracle, trellis_ref as ref
from strix_trellis_b200 import native as N, synthetic
from gpu_util import dev, gate, host

pytestmark = pytest.mark.gpu


def oracle_linear(layer, x, alpha=1.0, beta=0.0, old=None):
    return c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, layer.bits, 2, x, alpha, beta, old)


def view_desc(t):
    nbytes = ((t.shape[0] - 1) * t.stride(0) + t.shape[1]) * 4
    return N.tensor_desc(t.data_ptr(), nbytes, tuple(t.shape), (t.stride(0), t.stride(1)))


def cur_stream():
    from strix_trellis_b200.runtime import _cur_stream
    return _cur_stream(None)


@pytest.fixture(scope="module")
def ctx():
    from strix_trellis_b200.runtime import Context
    c = Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


@pytest.mark.parametrize("creator", ["plain", "tiled", "splitk", "r1"])
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_dense_plan_on_strided_views(ctx, creator, rows):
    lib = ctx.lib
    layer = synthetic.make_layer(1024, 640, 4, 9500, bias=True)
    w = ctx.prepare(layer)
    x = synthetic.make_activations(rows, 1024, seed=9501)
    old = synthetic.rng_for(9502).normal(0, 0.5, (rows, 640)).astype(np.float32)
    # the activation is a column slice of a wider buffer, the output a slice of a wider one
    xbuf = torch.full((rows, 1024 + 256), float("nan"), device="cuda")
    ybuf = torch.full((rows, 640 + 128), 7.0, device="cuda")
    xv, yv = xbuf[:, 128:128 + 1024], ybuf[:, 128:]
    xv.copy_(dev(x))
    yv.copy_(dev(old))
    d = w.matmul_desc(xv, yv, alpha=0.75, beta=-0.5)
    need = N.u64(0)
    N.check(lib.strix_tp_dense_workspace_bytes(ctx.handle, C.byref(d), 0, C.byref(need)), "workspace")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    if creator in ("splitk", "r1"):  # the plain and tiled creators take no workspace: scratch is the library's
        d.workspace, d.workspace_bytes = ws.data_ptr(), need.value
    sd, plan = cur_stream(), N.vp()
    if creator == "plain":
        st = lib.strix_tp_dense_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan))
    elif creator == "tiled":
        st = lib.strix_tp_dense_plan_create_tiled(ctx.handle, C.byref(d), C.byref(sd), min(4, rows), C.byref(plan))
    elif creator == "splitk":
        st = lib.strix_tp_dense_plan_create_splitk(ctx.handle, C.byref(d), C.byref(sd), min(4, rows), 1, C.byref(plan))
    else:
        need2 = N.u64(0)
        N.check(lib.strix_tp_dense_r1_workspace_bytes(ctx.handle, C.byref(d), 1, 0, C.byref(need2)), "r1 workspace")
        ws = torch.empty(max(need2.value, 256), dtype=torch.uint8, device="cuda")
        d.workspace, d.workspace_bytes = ws.data_ptr(), need2.value
        st = lib.strix_tp_dense_plan_create_r1(ctx.handle, C.byref(d), C.byref(sd), 1, 0, C.byref(plan))
    N.check(st, "dense plan create " + creator)
    N.check(lib.strix_tp_dense_plan_submit(plan), "submit")
    torch.cuda.synchronize()
    gate(host(yv), oracle_linear(layer, x, 0.75, -0.5, old), f"dense plan {creator} rows={rows}")
    assert (host(ybuf[:, :128]) == 7.0).all()  # nothing outside the view is written
    # a second submit accumulates through beta again, from the current contents
    again = host(yv).copy()
    N.check(lib.strix_tp_dense_plan_submit(plan), "submit")
    torch.cuda.synchronize()
    gate(host(yv), oracle_linear(layer, x, 0.75, -0.5, again), f"dense plan {creator} second submit")
    assert lib.strix_weights_destroy(w.handle) == N.INVALID_ARGUMENT  # retained by the plan
    N.check(lib.strix_tp_dense_plan_destroy(plan), "destroy")
    w.close()


def test_dense_plan_rejects_bad_views(ctx):
    lib = ctx.lib
    layer = synthetic.make_layer(256, 256, 2, 9510)
    w = ctx.prepare(layer)
    sd, plan = cur_stream(), N.vp()
    x9, y9 = torch.zeros((9, 256), device="cuda"), torch.zeros((9, 256), device="cuda")
    d = w.matmul_desc(x9, y9)
    assert lib.strix_tp_dense_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan)) != N.SUCCESS
    x, y = torch.zeros((2, 256), device="cuda"), torch.zeros((2, 256), device="cuda")
    d = w.matmul_desc(x, y)
    d.output.strides[0] = 128  # rows overlap
    assert lib.strix_tp_dense_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan)) != N.SUCCESS
    d = w.matmul_desc(x, y)
    d.input.strides[1] = 2  # channel stride must be one
    assert lib.strix_tp_dense_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan)) != N.SUCCESS
    d = w.matmul_desc(x, x)  # aliased input and output
    assert lib.strix_tp_dense_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan)) == N.INVALID_ARGUMENT
    w.close()


@pytest.mark.parametrize("rows", [1, 6])
def test_pair_plan(ctx, rows):
    lib = ctx.lib
    a = synthetic.make_layer(768, 384, 3, 9520, bias=True)
    b = synthetic.make_layer(768, 256, 5, 9521)
    wa, wb = ctx.prepare(a), ctx.prepare(b)
    x = synthetic.make_activations(rows, 768, seed=9522)
    old = synthetic.rng_for(9523).normal(0, 0.5, (rows, 256)).astype(np.float32)
    xd, ya, yb = dev(x), torch.zeros((rows, 384), device="cuda"), dev(old.copy())
    d = N.PairDesc()
    lib.strix_tp_dense_pair_desc_init(C.byref(d))
    d.input = view_desc(xd)
    d.member[0].weights, d.member[0].output, d.member[0].alpha, d.member[0].beta = wa.handle, view_desc(ya), 1.0, 0.0
    d.member[1].weights, d.member[1].output, d.member[1].alpha, d.member[1].beta = wb.handle, view_desc(yb), 2.0, 1.0
    need = N.u64(0)
    N.check(lib.strix_tp_dense_pair_workspace_bytes(ctx.handle, C.byref(d), C.byref(need)), "pair workspace")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = ws.data_ptr(), need.value
    sd, plan = cur_stream(), N.vp()
    N.check(lib.strix_tp_dense_pair_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan)), "pair create")
    N.check(lib.strix_tp_dense_pair_plan_submit(plan), "pair submit")
    torch.cuda.synchronize()
    gate(host(ya), oracle_linear(a, x), "pair member 0")
    gate(host(yb), oracle_linear(b, x, 2.0, 1.0, old), "pair member 1")
    N.check(lib.strix_tp_dense_pair_plan_destroy(plan), "pair destroy")
    wa.close()
    wb.close()


@pytest.mark.parametrize("rows", [1, 8])
def test_swiglu_plan(ctx, rows):
    lib = ctx.lib
    g = synthetic.make_layer(512, 384, 4, 9530, sigma=0.5, bias=True)
    u = synthetic.make_layer(512, 384, 3, 9531, sigma=0.5)
    wg, wu = ctx.prepare(g), ctx.prepare(u)
    x = synthetic.make_activations(rows, 512, seed=9532)
    xd = dev(x)
    hbuf = torch.full((rows, 512), -3.0, device="cuda")
    hv = hbuf[:, 128:]
    dg, du = torch.zeros((rows, 384), device="cuda"), torch.zeros((rows, 384), device="cuda")
    d = N.SwigluDesc()
    lib.strix_tp_swiglu_desc_init(C.byref(d))
    d.input, d.gate, d.up, d.hidden_output = view_desc(xd), wg.handle, wu.handle, view_desc(hv)
    d.diagnostic_gate, d.diagnostic_up, d.diagnostic_bytes = dg.data_ptr(), du.data_ptr(), rows * 384 * 4
    need = N.u64(0)
    N.check(lib.strix_tp_swiglu_workspace_bytes(ctx.handle, C.byref(d), C.byref(need)), "swiglu workspace")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = ws.data_ptr(), need.value
    sd, plan = cur_stream(), N.vp()
    N.check(lib.strix_tp_swiglu_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan)), "swiglu create")
    N.check(lib.strix_tp_swiglu_plan_submit(plan), "swiglu submit")
    torch.cuda.synchronize()
    gate_ref, up_ref = oracle_linear(g, x), oracle_linear(u, x)
    gate(host(dg), gate_ref, "swiglu gate diagnostic")
    gate(host(du), up_ref, "swiglu up diagnostic")
    # the activation applied to this library's own gate/up is exact to the contract's formula
    np.testing.assert_allclose(host(hv), ref.swiglu(host(dg), host(du)), rtol=2e-6, atol=1e-30)
    gate(host(hv), ref.swiglu(gate_ref, up_ref), "swiglu hidden", rel_bound=5e-3, nrmse_bound=1e-4)
    assert (host(hbuf[:, :128]) == -3.0).all()
    N.check(lib.strix_tp_swiglu_plan_destroy(plan), "swiglu destroy")
    wg.close()
    wu.close()


@pytest.mark.parametrize("rows,groups", [(1, 8), (4, 3)])
def test_grouped_gemv_plan(ctx, rows, groups):
    lib = ctx.lib
    layers = [synthetic.make_layer(256, 384, 4, 9540 + i, bias=(i % 2 == 0)) for i in range(groups)]
    ws_ = [ctx.prepare(l) for l in layers]
    xs = [synthetic.make_activations(rows, 256, seed=9550 + i) for i in range(groups)]
    in_stride, out_stride = groups * 256 + 128, groups * 384
    xbuf = torch.zeros((rows, in_stride), device="cuda")
    ybuf = torch.full((rows, out_stride), float("nan"), device="cuda")
    for i in range(groups):
        xbuf[:, i * 256:(i + 1) * 256] = dev(xs[i])
    handles = (N.vp * groups)(*[w.handle for w in ws_])
    d = N.GroupedGemvDesc()
    d.struct_size, d.abi_version = C.sizeof(N.GroupedGemvDesc), N.ABI_VERSION
    d.weights, d.group_count, d.rows = C.cast(handles, C.POINTER(N.vp)), groups, rows
    d.flags = 1  # STRIX_GEMV_ROW_INVARIANT_R1, the only accepted contract
    d.input, d.input_row_stride, d.input_group_stride = xbuf.data_ptr(), in_stride, 256
    d.input_buffer_bytes = xbuf.numel() * 4
    d.output, d.output_row_stride, d.output_group_stride = ybuf.data_ptr(), out_stride, 384
    d.output_buffer_bytes = ybuf.numel() * 4
    need = N.u64(0)
    N.check(lib.strix_grouped_gemv_workspace_bytes(ctx.handle, C.byref(d), C.byref(need)), "grouped workspace")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = ws.data_ptr(), need.value
    sd, plan = cur_stream(), N.vp()
    N.check(lib.strix_grouped_gemv_plan_create(ctx.handle, C.byref(d), C.byref(sd), C.byref(plan)), "grouped create")
    N.check(lib.strix_grouped_gemv_plan_submit(plan), "grouped submit")
    torch.cuda.synchronize()
    got = host(ybuf)
    for i in range(groups):
        gate(got[:, i * 384:(i + 1) * 384], oracle_linear(layers[i], xs[i]), f"grouped gemv group {i}")
    N.check(lib.strix_grouped_gemv_plan_destroy(plan), "grouped destroy")
    for w in ws_:
        w.close()


def test_pre_routed_grouped_call(ctx):
    lib = ctx.lib
    layers = [synthetic.make_layer(512, 256, 2 + i, 9560 + i, bias=True) for i in range(3)]
    ws_ = [ctx.prepare(l) for l in layers]
    counts = [2, 0, 5]  # an expert with no token is legal
    xs = [synthetic.make_activations(max(c, 1), 512, seed=9570 + i)[:c] for i, c in enumerate(counts)]
    xd = [dev(x) if len(x) else torch.zeros((0, 512), device="cuda") for x in xs]
    yd = [torch.zeros((c, 256), device="cuda") for c in counts]
    groups = (N.MatmulDesc * 3)()
    for i in range(3):
        groups[i] = ws_[i].matmul_desc(xd[i], yd[i])
    d = N.GroupedMoeDesc()
    d.struct_size, d.abi_version = C.sizeof(N.GroupedMoeDesc), N.ABI_VERSION
    d.groups, d.group_count = groups, 3
    need = N.u64(0)
    N.check(lib.strix_grouped_moe_workspace_bytes(ctx.handle, C.byref(d), C.byref(need)), "grouped moe workspace")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = ws.data_ptr(), need.value
    sd = cur_stream()
    N.check(lib.strix_grouped_moe(ctx.handle, C.byref(d), C.byref(sd)), "grouped moe")
    torch.cuda.synchronize()
    for i, c in enumerate(counts):
        if c:
            gate(host(yd[i]), oracle_linear(layers[i], xs[i]), f"pre-routed group {i}")
    for w in ws_:
        w.close()


def test_weights_from_container_slices(ctx, tmp_path):
    """A safetensors file written to disk, loaded through the container reader, partitioned
    and prepared: the shard on the GPU computes what the CPU contract computes from the same
    sliced arrays."""
    from strix_trellis_b200 import container, tp
    layer = synthetic.make_layer(512, 640, 4, 9580, bias=True)
    from test_container_tp import write_file
    path = tmp_path / "layer.safetensors"
    write_file(path, {
        "blk.w.trellis": layer.trellis.view(np.int16), "blk.w.suh": layer.suh, "blk.w.svh": layer.svh,
        "blk.w.bias": layer.bias.astype(np.float32),
        "blk.w.mul1": np.array([0x83DCD12D], dtype=np.uint32).view(np.int32)})
    tensor = container.load_exl3(path, "blk.w")
    if True:
        x = synthetic.make_activations(2, 512, seed=9581)
        for axis, world in (("output", 2), ("input", 2)):
            for rank in range(world):
                part = tp.rank_partition(tensor, axis, rank, world)
                w = ctx.prepare(part)
                a0, a1 = tp.h128_bounds(512, world)[rank] if axis == "input" else (0, 512)
                xs = np.ascontiguousarray(x[:, a0:a1])
                got = host(w.gemv(dev(xs)))
                bias = None if part.bias is None else np.asarray(part.bias, np.float32)
                want = c_oracle.linear(np.ascontiguousarray(part.trellis).view(np.uint16), np.asarray(part.suh),
                                       np.asarray(part.svh), bias, 4, 2, xs)
                gate(got, want, f"{axis} shard {rank}")
                w.close()
