"""Tensor- and expert-parallel layers on the GPU.  With one GPU the ranks of a partition run
one after another on the same device and their results are recombined with the math the
collective performs (sum / concatenation); with two or more GPUs the same layers also run as
one process per GPU over NCCL."""
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


# ---- one process per GPU over NCCL ---------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_rank(rank, world, port, out):
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
    y_row = row.forward(xd).cpu().numpy()
    col = ColumnParallelLinear(ctx, as_tensor(layer), rank, world)
    y_col = col.forward(xd).cpu().numpy()
    model, inter, n_exp, tokens, top_k = 512, 256, 8, 6, 4
    layers = make_experts(n_exp, model, inter, 9300)
    per = -(-n_exp // world)
    mine = layers[rank * per:(rank + 1) * per]
    ws = [tuple(ctx.prepare(l[k]) for k in ("gate", "up", "down")) for l in mine]
    xm = synthetic.make_activations(tokens, model, seed=9301)
    ids, scores = synthetic.make_routes(tokens, n_exp, top_k, seed=9302)
    scores[2, 1] = 0.0
    home = [t for t in range(tokens) if t % world == rank]  # tokens live round-robin on the ranks
    ep = ExpertParallelMoE(ctx, ws, n_exp, rank, world, model, max_tokens=tokens, top_k=top_k)
    y_ep = ep.forward(torch.from_numpy(xm[home]).cuda(), ids[home].astype(np.int64), scores[home]).cpu().numpy()
    torch.cuda.synchronize()
    status = ctx.device_status()
    np.savez(out + f".{rank}.npz", y_row=y_row, y_col=y_col, y_ep=y_ep, home=np.array(home), status=status)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_over_nccl(tmp_path):
    import torch.multiprocessing as mp
    world, out = 2, str(tmp_path / "rank")
    mp.spawn(_nccl_rank, args=(world, _free_port(), out), nprocs=world, join=True)
    layer = synthetic.make_layer(1024, 768, 4, 9400, bias=True)
    x = synthetic.make_activations(4, 1024, seed=9401)
    want = oracle_linear(layer, x)
    model, inter, n_exp, tokens, top_k = 512, 256, 8, 6, 4
    layers = make_experts(n_exp, model, inter, 9300)
    xm = synthetic.make_activations(tokens, model, seed=9301)
    ids, scores = synthetic.make_routes(tokens, n_exp, top_k, seed=9302)
    scores[2, 1] = 0.0
    want_ep, _ = oracle_block(xm, layers, ids, scores, 1.0, 0.0, np.zeros((tokens, model), np.float32))
    got_ep = np.zeros_like(want_ep)
    for rank in range(world):
        r = np.load(out + f".{rank}.npz")
        assert int(r["status"]) == 0
        gate(r["y_row"], want, f"row-parallel all-reduce, rank {rank}")
        gate(r["y_col"], want, f"column-parallel all-gather, rank {rank}")
        got_ep[r["home"]] = r["y_ep"]
    gate(got_ep, want_ep, "expert-parallel all-to-all", MOE_REL, MOE_NRMSE)
