"""Tensor- and expert-parallel layers on the GPU.  With one GPU the ranks of a partition run
one after another on the same device and their results are recombined with the math the
exchange performs (sum / concatenation); with two or more GPUs the same layers also run as
one process per GPU, meeting through peer memory over NVLink (torch.distributed only carries
the arena handles at set-up)."""
import os
import socket
import numpy as np
import pytest
import torch

from oracle import c_oracle
from strix_trellis_b200 import synthetic, tp
from strix_trellis_b200.container import Exl3Tensor
from gpu_util import dev, gate, host
from test_gpu_moe import MOE_NRMSE, MOE_REL, make_experts, oracle_block

pytestmark = pytest.mark.gpu


def as_tensor(layer):
    return Exl3Tensor(layer.trellis, layer.suh, layer.svh, float(layer.bits), layer.codebook, layer.bias, "synthetic", "w")


def oracle_linear(layer, x):
    return c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, layer.bits, 2, x)


@pytest.fixture(scope="module")
def ctx():
    from strix_trellis_b200.runtime import Context
    c = Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("rows", [1, 5])
def test_row_parallel_shards_sum_to_the_layer(ctx, world, rows):
    from strix_trellis_b200.tp_runtime import RowParallelLinear
    layer = synthetic.make_layer(1536, 512, 4, 9100 + world, bias=True)
    x = synthetic.make_activations(rows, 1536, seed=9101)
    xd = dev(x)
    total = torch.zeros((rows, 512), device="cuda")
    want = np.zeros((rows, 512), np.float32)
    for rank in range(world):
        shard = RowParallelLinear(ctx, as_tensor(layer), rank, world, bias_rank=world - 1)
        local = host(shard.local(xd))
        a0, a1 = shard.bounds[rank]
        part = tp.rank_partition(as_tensor(layer), "input", rank, world, bias_rank=world - 1)
        ref = c_oracle.linear(np.ascontiguousarray(part.trellis), part.suh, part.svh, part.bias, layer.bits, 2,
                              np.ascontiguousarray(x[:, a0:a1]))
        gate(local, ref, f"row shard {rank}/{world}")
        want += ref
        total += dev(local)
        shard.close()
    gate(host(total), want, "row-parallel sum")


@pytest.mark.parametrize("world", [2, 3])
def test_column_parallel_shards_concatenate_to_the_layer(ctx, world):
    from strix_trellis_b200.tp_runtime import ColumnParallelLinear
    layer = synthetic.make_layer(512, 128 * 7, 3, 9200 + world, bias=True)  # 7 blocks: uneven shards
    x = synthetic.make_activations(3, 512, seed=9201)
    xd = dev(x)
    pieces = []
    for rank in range(world):
        shard = ColumnParallelLinear(ctx, as_tensor(layer), rank, world)
        pieces.append(host(shard.local(xd)))
        assert pieces[-1].shape[1] == shard.widths[rank]
        shard.close()
    got = np.concatenate(pieces, axis=1)
    gate(got, oracle_linear(layer, x), "column-parallel concat")
    full = ctx.prepare(layer)
    gate(got, host(full.gemv(xd)), "column shards vs the unsharded layer")
    full.close()


def test_expert_parallel_single_rank_matches_the_block(ctx):
    from strix_trellis_b200.tp_runtime import ExpertParallelMoE
    model, inter, n_exp, tokens, top_k = 512, 256, 8, 6, 4
    layers = make_experts(n_exp, model, inter, 9300)
    ws = [tuple(ctx.prepare(l[k]) for k in ("gate", "up", "down")) for l in layers]
    x = synthetic.make_activations(tokens, model, seed=9301)
    ids, scores = synthetic.make_routes(tokens, n_exp, top_k, seed=9302)
    scores[2, 1] = 0.0
    want, _ = oracle_block(x, layers, ids, scores, 1.0, 0.0, np.zeros((tokens, model), np.float32))
    ep = ExpertParallelMoE(ctx, ws, n_exp, 0, 1, model, max_tokens=tokens, top_k=top_k)
    y = ep.forward(dev(x), ids.astype(np.int64), scores)
    torch.cuda.synchronize()
    gate(host(y), want, "expert-parallel (1 rank)", MOE_REL, MOE_NRMSE)
    # the same routes through the plain device-routed plan: identical bits (same kernels, same order)
    from strix_trellis_b200.runtime import MoePlan
    y2 = torch.zeros((tokens, model), device="cuda")
    plan = MoePlan(ctx, ws, dev(x), y2, dev(ids.astype(np.uint32).view(np.int32)).view(torch.int32), dev(scores),
                   device_routed=True)
    plan.submit()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(y), host(y2))
    # the same forward frozen into a graph, fed through its static buffers
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ep2 = ExpertParallelMoE(ctx, ws, n_exp, 0, 1, model, max_tokens=tokens, top_k=top_k)
        run = ep2.capture(tokens)
        y3 = run(dev(x), dev(ids.astype(np.int64)), dev(scores))
        stream.synchronize()
    np.testing.assert_array_equal(host(y3), host(y2))
    ep2.close()
    plan.close()
    ep.close()
    for t in ws:
        for w in t:
            w.close()


def test_layers_follow_the_callers_stream(ctx):
    """A plan is frozen on the stream it was created for.  A dense layer used from another
    stream builds a plan for that stream (kernels and their consumers stay ordered); the
    expert-parallel layer, whose step is one frozen sequence, refuses another stream."""
    from strix_trellis_b200.tp_runtime import ExpertParallelMoE, RowParallelLinear
    layer = synthetic.make_layer(1024, 512, 4, 9500, bias=True)
    x = synthetic.make_activations(2, 1024, seed=9501)
    want = oracle_linear(layer, x)
    row = RowParallelLinear(ctx, as_tensor(layer), 0, 1)
    xd = dev(x)
    y = torch.zeros((2, 512), device="cuda")
    gate(host(row.forward(xd, y)), want, "default stream")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        y.fill_(float("nan"))            # ordered before the layer only if the layer runs on `side`
        row.forward(xd, y)
        got = y.clone()
    side.synchronize()
    gate(host(got), want, "side stream")
    assert len(row.plans) == 2
    row.close()
    model, inter, n_exp = 256, 128, 4
    layers = make_experts(n_exp, model, inter, 9510)
    ws = [tuple(ctx.prepare(l[k]) for k in ("gate", "up", "down")) for l in layers]
    ep = ExpertParallelMoE(ctx, ws, n_exp, 0, 1, model, max_tokens=2, top_k=2)
    with torch.cuda.stream(side):
        with pytest.raises(RuntimeError):
            ep.run(1)
    ep.close()
    for t in ws:
        for w in t:
            w.close()


# ---- one process per GPU, exchanges through peer memory ---------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _peer_rank(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from strix_trellis_b200.runtime import Context
    from strix_trellis_b200.tp_runtime import ColumnParallelLinear, ExpertParallelMoE, RowParallelLinear
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = Context(rank)
    layer = synthetic.make_layer(1024, 768, 4, 9400, bias=True)
    x = synthetic.make_activations(4, 1024, seed=9401)
    xd = torch.from_numpy(x).cuda()
    row = RowParallelLinear(ctx, as_tensor(layer), rank, world)
    y_row = [row.forward(xd).cpu().numpy() for _ in range(3)][-1]  # regions are reused with alternating parity
    col = ColumnParallelLinear(ctx, as_tensor(layer), rank, world)
    y_col = [col.forward(xd).cpu().numpy() for _ in range(3)][-1]
    model, inter, n_exp, tokens, top_k = 512, 256, 8, 6, 4
    layers = make_experts(n_exp, model, inter, 9300)
    per = -(-n_exp // world)
    mine = layers[rank * per:(rank + 1) * per]
    ws = [tuple(ctx.prepare(l[k]) for k in ("gate", "up", "down")) for l in mine]
    xm = synthetic.make_activations(tokens, model, seed=9301)
    ids, scores = synthetic.make_routes(tokens, n_exp, top_k, seed=9302)
    scores[2, 1] = 0.0
    ids = ids.astype(np.int64)
    ids[5, 1] = n_exp + 9  # an id outside the id space: that token's row must come out NaN, nothing else changes
    slots = -(-tokens // world)
    home = list(range(rank * slots, min(tokens, (rank + 1) * slots)))  # tokens live rank-major
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ep = ExpertParallelMoE(ctx, ws, n_exp, rank, world, model, max_tokens=slots, top_k=top_k)
        y_ep = ep.forward(torch.from_numpy(xm[home]).cuda(), ids[home], scores[home]).cpu().numpy()
        # the same step frozen into a graph on every rank
        run = ep.capture(len(home))
        y_graph = run(torch.from_numpy(xm[home]).cuda(), ids[home], scores[home]).cpu().numpy()
        stream.synchronize()
    torch.cuda.synchronize()
    status = ctx.device_status()
    np.savez(out + f".{rank}.npz", y_row=y_row, y_col=y_col, y_ep=y_ep, y_graph=y_graph, home=np.array(home),
             status=status)
    dist.barrier()
    ep.close()
    row.close()
    col.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_over_peer_memory(tmp_path):
    import torch.multiprocessing as mp
    world, out = 2, str(tmp_path / "rank")
    mp.spawn(_peer_rank, args=(world, _free_port(), out), nprocs=world, join=True)
    layer = synthetic.make_layer(1024, 768, 4, 9400, bias=True)
    x = synthetic.make_activations(4, 1024, seed=9401)
    want = oracle_linear(layer, x)
    model, inter, n_exp, tokens, top_k = 512, 256, 8, 6, 4
    layers = make_experts(n_exp, model, inter, 9300)
    xm = synthetic.make_activations(tokens, model, seed=9301)
    ids, scores = synthetic.make_routes(tokens, n_exp, top_k, seed=9302)
    scores[2, 1] = 0.0
    want_ep, _ = oracle_block(xm, layers, ids, scores, 1.0, 0.0, np.zeros((tokens, model), np.float32))
    got_ep, got_graph = np.zeros_like(want_ep), np.zeros_like(want_ep)
    rows = []
    for rank in range(world):
        r = np.load(out + f".{rank}.npz")
        assert int(r["status"]) == 0
        gate(r["y_row"], want, f"row-parallel sum, rank {rank}")
        gate(r["y_col"], want, f"column-parallel concatenation, rank {rank}")
        rows.append(r["y_row"])
        got_ep[r["home"]] = r["y_ep"]
        got_graph[r["home"]] = r["y_graph"]
    assert rows[0].tobytes() == rows[1].tobytes()  # rank-ordered sum: the same bits on every rank
    assert np.isnan(got_ep[5]).all()               # the token with an id outside the id space
    gate(got_ep[:5], want_ep[:5], "expert-parallel block", MOE_REL, MOE_NRMSE)
    assert got_graph[:5].tobytes() == got_ep[:5].tobytes() and np.isnan(got_graph[5]).all()


def _absent_peer_rank(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from strix_trellis_b200.peer import PeerGroup
    from strix_trellis_b200.runtime import Context
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = Context(rank)
    count = 2048
    group = PeerGroup(ctx, 1 << 20, rank=rank, world=world)
    region = group.reserve(world * count * 8)
    group.set_wait_polls(1 << 16)  # a tenth of a second instead of several
    rows = torch.full((count,), float(rank + 1), device="cuda")
    late = 0
    if rank == 0:  # rank 1 never joins this exchange: nothing sets the words rank 0 waits for
        group.sum_rows([rows], region)
        torch.cuda.synchronize()
        late = ctx.device_status()
    dist.barrier()  # rank 1 was idle meanwhile: it has nothing in flight
    untouched = bool((rows == float(rank + 1)).all().item())
    group.close()
    # the context is still usable: a fresh group's exchange completes on both ranks
    again = PeerGroup(ctx, 1 << 20, rank=rank, world=world)
    region = again.reserve(world * count * 8)
    again.sum_rows([rows], region)
    torch.cuda.synchronize()
    np.savez(out + f".{rank}.npz", late=late, untouched=untouched, total=rows.cpu().numpy(), after=ctx.device_status())
    again.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_a_peer_that_never_arrives_is_reported_and_the_context_survives(tmp_path):
    """Failure detection without a fault: one rank simply does not take part in an exchange.  The
    other rank's wait runs out after its (shortened) limit, bit 5 of its device status word says
    so, its rows are left as they were, and after the group has been replaced both ranks
    exchange normally again."""
    import torch.multiprocessing as mp
    world, out = 2, str(tmp_path / "rank")
    mp.spawn(_absent_peer_rank, args=(world, _free_port(), out), nprocs=world, join=True)
    r0, r1 = (np.load(out + f".{rank}.npz") for rank in range(world))
    assert int(r0["late"]) == 32 and int(r1["late"]) == 0
    assert bool(r0["untouched"]) and bool(r1["untouched"])
    for r in (r0, r1):
        assert int(r["after"]) == 0
        assert (r["total"] == 3.0).all()
