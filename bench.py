#!/usr/bin/env python3
"""Benchmark of the fused trellis decode-GEMV (the headline metric) on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N=1): benchmark configuration 2 restricted to the rate and row count the
metric names -- K=4 bits/weight, one activation row -- over its four shapes
(4096x4096, 5120x5120, 1152x4096, 4096x14336), seeded synthetic weights.  A "step" is
one launch of each of 24 device copies of each shape (96 launches, 1.28 GB of packed
weights, ten times L2), so weights always come from HBM.  `value` is packed weight
bytes per second (the reference's own definition, README.md:224-226) with inputs
resident on the device and every call captured in one CUDA graph.  `e2e` is the same
metric through the public C-ABI call (strix_linear_plan_submit) with HOST activations:
the step's activation rows are copied from pinned host memory before its calls and the
output rows copied back to pinned host memory after them, inside the timed region.

With N>1 (launched under torchrun) every rank runs the same workload on its own GPU
(replicas: the plain GEMV has no cross-GPU exchange) and the value is the sum.

`extra` in the JSON line carries the other configurations of the metric, measured outside
the timed region: rates x rows on the largest shape, the prefill GEMM (K4/K5/K6), the
routed-expert block on one rank's bank, and at every N the tensor-parallel dense layers
(row-parallel + all-reduce, LM head + all-gather) and the expert-parallel block
(all-to-all dispatch and return).  `--no-extra` skips them; `--case gemv|gemm|gemm-small|moe|decode` runs one
small fixed workload of one kernel for profilers.

`--impl reference` times the CPU contract (this repository's C restatement of the
reference's NumPy path, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [(4096, 4096), (5120, 5120), (1152, 4096), (4096, 14336)]
BITS, ROWS = 4, 1
CLONES = 24  # device copies per shape: 24 x (8.4 + 13.1 + 2.4 + 29.4) MB = 1.28 GB per step
METRIC = "K4 R1 decode-GEMV GB/s over packed weight bytes"
WORKLOAD = "config2: K4 R1 fused decode-GEMV sweep over (4096,4096),(5120,5120),(1152,4096),(4096,14336)"


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_baseline(seconds_budget=12.0):
    """C restatement of the reference CPU contract, all host threads, on a sample: whole
    K4 R1 layers of the smallest two shapes, repeated until the budget is spent."""
    from oracle import c_oracle
    from strix_trellis_b200 import synthetic
    c_oracle.build()
    layers = [synthetic.make_layer(i, n, BITS, seed=synthetic.BASE_SEED + k)
              for k, (i, n) in enumerate([(1152, 4096), (4096, 4096)])]
    xs = [synthetic.make_activations(ROWS, layer.inputs) for layer in layers]
    for layer, x in zip(layers, xs):
        c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, BITS, 2, x)
    done_bytes, calls, t0 = 0, 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds_budget:
        for layer, x in zip(layers, xs):
            c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, BITS, 2, x)
            done_bytes += layer.packed_bytes
            calls += 1
    dt = time.perf_counter() - t0
    return {"value": done_bytes / dt / 1e9, "unit": "GB/s", "cores": c_oracle.threads(), "kind": "port",
            "sample": f"{calls} whole K4 R1 layers of shapes (1152,4096),(4096,4096) in {dt:.1f} s"}, dt / max(calls, 1)


def numpy_baseline():
    """The NumPy restatement of the reference's CPU path (vectorised decode + staged float32
    contract) on one 1152 x 4096 K4 layer, one row, one process: the figure the reference's own
    Python model would give on this host."""
    from oracle import trellis_ref as ref
    from strix_trellis_b200 import synthetic
    layer = synthetic.make_layer(1152, 4096, BITS, seed=synthetic.BASE_SEED + 2)
    x = synthetic.make_activations(ROWS, 1152)
    t0 = time.perf_counter()
    ref.linear_stages(x, layer.trellis, layer.suh, layer.svh, BITS, "mul1", None)
    dt = time.perf_counter() - t0
    return {"value": layer.packed_bytes / dt / 1e9, "unit": "GB/s", "cores": 1,
            "sample": f"one 1152x4096 K4 R1 layer through oracle/trellis_ref.py in {dt:.2f} s"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1; the CPU arm uses every core this process may run on
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    per_step = []
    base = None
    budget = max(2.0, 20.0 / max(args.steps + args.warmup, 1))
    for _ in range(args.warmup + args.steps):
        base, _ = cpu_baseline(seconds_budget=budget)
        per_step.append(base["value"])
    vals = per_step[args.warmup:]
    value = float(np.mean(vals))
    base["value"] = value
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(budget * 1e3, 1), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 weights, f32 accumulate",
            "data": "synthetic", "config": {"workload": WORKLOAD, "host": "CPU contract, all host threads"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def time_calls(torch, stream, fn, reps, warm=3):
    """Average device time of fn() in microseconds: CUDA events on the launching stream."""
    with torch.cuda.stream(stream):
        for _ in range(warm):
            fn()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            fn()
        b.record(stream)
        stream.synchronize()
    return a.elapsed_time(b) * 1e3 / reps


def gemv_sweep(torch, ctx, stream, shape=(4096, 14336), rates=(2, 3, 4, 5, 6), rows_list=(1, 8), copies=12):
    """Rates and row counts of benchmark configuration 2 on its largest shape: microseconds per
    launch and GB/s over packed bytes, `copies` device copies launched in turn as one graph
    (12 x 14.7 MB at K2 is already larger than L2)."""
    from strix_trellis_b200 import native as N, synthetic
    out = {}
    for bits in rates:
        layer = synthetic.make_layer(shape[0], shape[1], bits, seed=synthetic.BASE_SEED + 800 + bits)
        ws = [ctx.prepare(layer) for _ in range(copies)]
        for rows in rows_list:
            x = torch.from_numpy(synthetic.make_activations(rows, shape[0], seed=synthetic.BASE_SEED + 801)).cuda()
            y = torch.empty((rows, shape[1]), dtype=torch.float32, device="cuda")
            with torch.cuda.stream(stream):
                plans = [w.plan(x, y, N.OP_GEMV, stream=stream) for w in ws]
                for p in plans:
                    p.submit()
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for p in plans:
                        p.submit()
            us = time_calls(torch, stream, graph.replay, 5) / copies
            out[f"K{bits}_R{rows}"] = {"us": round(us, 2), "GBps": round(layer.packed_bytes / us / 1e3, 1)}
            del graph
            for p in plans:
                p.close()
        for w in ws:
            w.close()
    return out


def gemm_case(torch, ctx, stream, rows_list, bits=4, inputs=4096, outputs=12288, reps=None):
    """Prefill GEMM of benchmark configuration 3 (4096 -> 12288): microseconds and TFLOP/s."""
    from strix_trellis_b200 import native as N, synthetic
    w = ctx.prepare(synthetic.make_layer(inputs, outputs, bits, seed=synthetic.BASE_SEED + 300 + bits))
    out = {}
    for m in rows_list:
        x = torch.from_numpy(synthetic.make_activations(m, inputs, seed=synthetic.BASE_SEED + 301)).cuda()
        y = torch.empty((m, outputs), dtype=torch.float32, device="cuda")
        ws = torch.empty(max(w.workspace_bytes(x, y), 256), dtype=torch.uint8, device="cuda")
        with torch.cuda.stream(stream):
            plan = w.plan(x, y, N.OP_GEMM, workspace=ws, stream=stream)
        us = time_calls(torch, stream, plan.submit, reps or (10 if m <= 2048 else 4))
        out[f"M{m}"] = {"us": round(us, 1), "TFLOPs": round(2.0 * m * inputs * outputs / us / 1e6, 1)}
        plan.close()
    w.close()
    return out


def moe_case(torch, ctx, stream, tokens_list, experts=32, top_k=8, model=4096, inter=2048, bits=2, reps=12):
    """Routed-expert block of benchmark configuration 5 on one rank's bank of `experts`
    experts (K2 gate/up/down, 201 MB of packed weights), device-routed.  Routes rotate over
    four seeded sets between submits (one small device copy, inside the timed region) so that
    successive submits read different experts.  Microseconds per submit and GB/s over the packed
    bytes of the DISTINCT experts a submit touches (an expert's weights are read once per eight
    rows routed to it)."""
    from strix_trellis_b200 import synthetic
    from strix_trellis_b200.runtime import MoePlan
    proto = [synthetic.make_layer(model, inter, bits, seed=synthetic.BASE_SEED + 500, sigma=0.5),
             synthetic.make_layer(model, inter, bits, seed=synthetic.BASE_SEED + 501, sigma=0.5),
             synthetic.make_layer(inter, model, bits, seed=synthetic.BASE_SEED + 502, sigma=0.5)]
    bank = [tuple(ctx.prepare(l) for l in proto) for _ in range(experts)]  # distinct device copies
    out = {}
    for t in tokens_list:
        x = torch.from_numpy(synthetic.make_activations(t, model, seed=synthetic.BASE_SEED + 503)).cuda()
        y = torch.zeros((t, model), dtype=torch.float32, device="cuda")
        sets = [synthetic.make_routes(t, experts, top_k, seed=synthetic.BASE_SEED + 504 + k) for k in range(4)]
        ids_all = [torch.from_numpy(i.astype(np.uint32).view(np.int32)).cuda() for i, _ in sets]
        sc_all = [torch.from_numpy(sc).cuda() for _, sc in sets]
        ids_d, sc_d = ids_all[0].clone(), sc_all[0].clone()
        with torch.cuda.stream(stream):
            plan = MoePlan(ctx, bank, x, y, ids_d, sc_d, device_routed=True, stream=stream)
        turn = [0]

        def submit():
            turn[0] = (turn[0] + 1) % 4
            ids_d.copy_(ids_all[turn[0]])
            sc_d.copy_(sc_all[turn[0]])
            plan.submit()
        us = time_calls(torch, stream, submit, reps)
        distinct = float(np.mean([len(np.unique(i)) for i, _ in sets]))
        unique_bytes = distinct * sum(l.packed_bytes for l in proto)
        out[f"T{t}"] = {"us": round(us, 1), "distinct_experts": round(distinct, 1),
                        "GBps_over_distinct_expert_bytes": round(unique_bytes / us / 1e3, 1)}
        plan.close()
    for e in bank:
        for w in e:
            w.close()
    return out


def _gates(got, want, what, nrmse_bound=3e-5):
    """The reference's acceptance criterion (docs/GPU_TESTS.md:126-131); returns the two figures."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    if not np.isfinite(got).all():
        raise SystemExit(f"{what}: non-finite output")
    err = np.abs(got - want)
    maxabs = float(err.max())
    nrmse = float(np.sqrt((err ** 2).sum() / max((want ** 2).sum(), 1e-30)))
    if maxabs > 5e-4 * max(1.0, float(np.abs(want).max())) or nrmse > nrmse_bound:
        raise SystemExit(f"{what}: parity check failed before timing (maxabs {maxabs:.3e}, NRMSE {nrmse:.3e})")
    return maxabs, nrmse


def _graph_us(torch, stream, calls, replays=6):
    """`calls` (a list of thunks, each a fixed sequence of kernel launches) captured into one
    CUDA graph; device time per call in microseconds over `replays` replays."""
    with torch.cuda.stream(stream):
        for c in calls:
            c()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for c in calls:
                c()
        graph.replay()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(replays):
            graph.replay()
        b.record(stream)
        stream.synchronize()
    return a.elapsed_time(b) * 1e3 / (replays * len(calls)), graph


def tp_case(torch, dist, ctx, stream, rank, world, rows_list=(1, 4, 8)):
    """Benchmark configuration 4 at `world` ranks: (a) row-parallel 16384 -> 4096 K5, rank outputs
    summed over the ranks, (b) LM head 4096 -> 129280 K5, rank blocks concatenated.  Each rank
    generates only its own shard and rotates over enough device copies of it to exceed L2 twice.
    Before timing every rank checks its result against the CPU contract: the sum of the ranks'
    shard outputs (each rank evaluates its own shard on the CPU, the references are added in
    float64 across ranks), its own block of the logits (first sixteen H128 blocks), and the bytes
    of every other rank's block against a hash taken where the block was computed.  Microseconds
    per call (local kernel + exchange, all copies in one CUDA graph) and for the local kernel
    alone, max over ranks."""
    import hashlib
    from oracle import c_oracle
    from strix_trellis_b200 import synthetic, tp
    from strix_trellis_b200.container import Exl3Tensor
    from strix_trellis_b200.tp_runtime import ColumnParallelLinear, RowParallelLinear

    def shard_layer(inputs, outputs, seed):
        layer = synthetic.make_layer(inputs, outputs, 5, seed=seed + rank)
        return Exl3Tensor(layer.trellis, layer.suh, layer.svh, 5.0, layer.codebook, None, "synthetic", "w"), layer

    a0, a1 = tp.h128_bounds(16384, world)[rank]
    bounds = tp.h128_bounds(129280, world)
    b0, b1 = bounds[rank]
    row_t, row_l = shard_layer(a1 - a0, 4096, synthetic.BASE_SEED + 600)
    col_t, col_l = shard_layer(4096, b1 - b0, synthetic.BASE_SEED + 700)
    need = 256 * 1024 * 1024
    with torch.cuda.stream(stream):
        rows_ = [RowParallelLinear(ctx, row_t, rank, world, full_inputs=16384)
                 for _ in range(-(-need // row_l.packed_bytes))]
        cols_ = [ColumnParallelLinear(ctx, col_t, rank, world, full_outputs=129280)
                 for _ in range(-(-need // col_l.packed_bytes))]
    out = {"row_parallel_copies": len(rows_), "lm_head_copies": len(cols_), "parity_checked": True}
    worst = {"row_parallel": [0.0, 0.0], "lm_head": [0.0, 0.0]}
    for r in rows_list:
        x_row_h = synthetic.make_activations(r, 16384, seed=synthetic.BASE_SEED + 601)
        x_col_h = synthetic.make_activations(r, 4096, seed=synthetic.BASE_SEED + 701)
        x_row, x_col = torch.from_numpy(x_row_h).cuda(), torch.from_numpy(x_col_h).cuda()
        ys = [torch.empty((r, 4096), dtype=torch.float32, device="cuda") for _ in rows_]
        # ---- parity before timing (first copy; the other copies hold the same bytes) ----
        with torch.cuda.stream(stream):
            got_row = rows_[0].forward(x_row, ys[0]).cpu().numpy()
            got_col_t = cols_[0].forward(x_col)
            got_col = got_col_t.cpu().numpy()
            local_block = cols_[0].local(x_col).cpu().numpy()
        want = c_oracle.linear(row_l.trellis, row_l.suh, row_l.svh, None, 5, 2,
                               np.ascontiguousarray(x_row_h[:, a0:a1])).astype(np.float64)
        want_t = torch.from_numpy(want).cuda()
        if world > 1:
            dist.all_reduce(want_t)
        m = _gates(got_row, want_t.cpu().numpy(), f"row-parallel sum, rank {rank}, rows {r}")
        worst["row_parallel"] = [max(a, b) for a, b in zip(worst["row_parallel"], m)]
        head = min(2048, b1 - b0)
        want_head = c_oracle.linear(np.ascontiguousarray(col_l.trellis[:, :head // 16]), col_l.suh, col_l.svh[:head],
                                    None, 5, 2, x_col_h)
        if world > 1:
            dist.barrier()
        m = _gates(got_col[:, b0:b0 + head], want_head, f"LM head block, rank {rank}, rows {r}")
        worst["lm_head"] = [max(a, b) for a, b in zip(worst["lm_head"], m)]
        digests = [hashlib.sha256(local_block.tobytes()).hexdigest()]
        if world > 1:
            digests = [None] * world
            dist.all_gather_object(digests, hashlib.sha256(local_block.tobytes()).hexdigest())
        for q, (c0, c1) in enumerate(bounds):
            if hashlib.sha256(np.ascontiguousarray(got_col[:, c0:c1]).tobytes()).hexdigest() != digests[q]:
                raise SystemExit(f"LM head: block of rank {q} arrived with different bytes on rank {rank}")
        # ---- timing: every copy once per graph replay ----
        us = [_graph_us(torch, stream, [lambda l=l, y=y: l.forward(x_row, y) for l, y in zip(rows_, ys)])[0],
              _graph_us(torch, stream, [lambda l=l, y=y: l.local(x_row, y) for l, y in zip(rows_, ys)])[0],
              _graph_us(torch, stream, [lambda l=l: l.forward(x_col) for l in cols_])[0],
              _graph_us(torch, stream, [lambda l=l: l.local(x_col) for l in cols_])[0]]
        t = torch.tensor(us, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = [round(float(v), 1) for v in t.tolist()]
        out[f"R{r}"] = {"row_parallel_us": us[0], "row_parallel_kernel_us": us[1],
                        "lm_head_us": us[2], "lm_head_kernel_us": us[3]}
    w = torch.tensor(worst["row_parallel"] + worst["lm_head"], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
    out["worst_maxabs_nrmse"] = {"row_parallel": [float(f"{v:.3e}") for v in w[:2].tolist()],
                                 "lm_head": [float(f"{v:.3e}") for v in w[2:].tolist()]}
    if world > 1:
        dist.barrier()
    for layer in rows_ + cols_:
        layer.close()
    return out


def ep_case(torch, dist, ctx, stream, rank, world, tokens_list=(1, 8, 64), experts=256, top_k=8, model=4096,
            inter=2048, bits=2, reps=6):
    """Benchmark configuration 5: 256 experts owned contiguously by the ranks, top-8 routing,
    K2 gate/up/down; tokens live rank-major on the ranks.  A step is two exchanges through
    peer memory around the expert kernels and the combine at the home rank in slot order.
    Every expert holds the same three seeded layers (distinct device copies), so before timing each
    rank checks its own tokens against the CPU contract evaluated with those layers (up to two
    tokens per rank).  Microseconds per step: the captured graph of one step replayed (device time,
    max over ranks) and the same step enqueued call by call.  Routes rotate over four seeded sets so
    that successive steps touch different experts."""
    from oracle import c_oracle
    from strix_trellis_b200 import synthetic
    from strix_trellis_b200.tp_runtime import ExpertParallelMoE
    proto = [synthetic.make_layer(model, inter, bits, seed=synthetic.BASE_SEED + 500, sigma=0.5),
             synthetic.make_layer(model, inter, bits, seed=synthetic.BASE_SEED + 501, sigma=0.5),
             synthetic.make_layer(inter, model, bits, seed=synthetic.BASE_SEED + 502, sigma=0.5)]
    per = -(-experts // world)
    mine = range(rank * per, min(experts, (rank + 1) * per))
    bank = [tuple(ctx.prepare(l) for l in proto) for _ in mine]
    out = {"parity_checked": True}
    worst = [0.0, 0.0]

    def lin(layer, v):
        return c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, bits, 2, v)

    with torch.cuda.stream(stream):
        for t in tokens_list:
            sets = [synthetic.make_routes(t, experts, top_k, seed=synthetic.BASE_SEED + 520 + k) for k in range(4)]
            x = synthetic.make_activations(t, model, seed=synthetic.BASE_SEED + 503)
            slots = -(-t // world)
            home = list(range(rank * slots, min(t, (rank + 1) * slots)))
            xh = torch.from_numpy(x[home]).cuda() if home else torch.zeros((0, model), device="cuda")
            ep = ExpertParallelMoE(ctx, bank, experts, rank, world, model, max_tokens=slots, top_k=top_k)
            on_device = [(torch.from_numpy(ids[home].astype(np.int64).reshape(len(home), top_k)).cuda(),
                          torch.from_numpy(scores[home].reshape(len(home), top_k)).cuda()) for ids, scores in sets]
            # ---- parity before timing ----
            got = ep.forward(xh, *on_device[0]).cpu().numpy()
            for j, token in enumerate(home[:2]):
                hidden = c_oracle.swiglu(lin(proto[0], x[token:token + 1]), lin(proto[1], x[token:token + 1]))
                down = lin(proto[2], hidden)[0]
                want = np.zeros(model, np.float32)
                for sc in sets[0][1][token]:  # ascending slot order from +0; every expert holds the same layers
                    if sc != 0.0:
                        want = want + np.float32(sc) * down
                # One token row whose eight slots hold the same expert layers: the slots' errors
                # (binary16 roundings of the hidden row that flip with the accumulation order) are
                # fully correlated, so a row's NRMSE scatters around the 8-token block figure the
                # tests hold to 2.5e-4; rows are held to twice that.  tests/test_gpu_moe.py takes
                # the block apart stage by stage at single-projection gates.
                m = _gates(got[j], want, f"expert-parallel block, token {token}, {t} tokens, rank {rank}", 5e-4)
                worst = [max(a, b) for a, b in zip(worst, m)]
            if world > 1:
                dist.barrier()  # the CPU check takes seconds on some ranks and nothing on others
            # ---- timing ----
            run = ep.capture(len(home))
            turn = [0]

            def step(fn):
                turn[0] = (turn[0] + 1) % 4
                return fn(xh, *on_device[turn[0]])
            us_graph = time_calls(torch, stream, lambda: step(run), reps if world == 1 else 2 * reps, warm=3)
            us_eager = time_calls(torch, stream, lambda: step(ep.forward), reps if world == 1 else 2 * reps, warm=3)
            tt = torch.tensor([us_graph, us_eager], device="cuda")
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            out[f"T{t}"] = {"us": round(float(tt[0].item()), 1), "us_call_by_call": round(float(tt[1].item()), 1)}
            if world > 1:
                dist.barrier()
            ep.close()
    w = torch.tensor(worst, device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
    out["worst_maxabs_nrmse"] = [float(f"{v:.3e}") for v in w.tolist()]
    for e in bank:
        for w_ in e:
            w_.close()
    return out


def run_case(args):
    """A small fixed workload of one kernel, for profilers: a few launches, inputs larger
    than L2, a few hundred MB on the device."""
    import torch
    from strix_trellis_b200 import native as N, synthetic
    from strix_trellis_b200.runtime import Context
    ctx = Context(0)
    stream = torch.cuda.Stream()
    if args.case == "gemv":
        layer = synthetic.make_layer(4096, 14336, BITS, seed=synthetic.BASE_SEED + 3)
        ws = [ctx.prepare(layer) for _ in range(8)]  # 8 x 29 MB: every launch reads cold weights
        x = torch.from_numpy(synthetic.make_activations(ROWS, 4096)).cuda()
        y = torch.empty((ROWS, 14336), dtype=torch.float32, device="cuda")
        with torch.cuda.stream(stream):
            plans = [w.plan(x, y, N.OP_GEMV, stream=stream) for w in ws]

        def one_pass():
            for p in plans:
                p.submit()
        us = time_calls(torch, stream, one_pass, 3, warm=1) / len(plans)
        print(json.dumps({"case": "gemv 4096x14336 K4 R1", "us_per_launch": round(us, 2),
                          "GBps": round(layer.packed_bytes / us / 1e3, 1), "status": ctx.device_status()}))
    elif args.case == "decode":
        # the decoder's own ceiling: decode + mma on tiles resident in shared memory, no memory traffic
        out = {"case": "decode-rate probe, 16 warps per SM (and 8 / 32 for K4), tiles in shared memory"}
        sm = torch.cuda.get_device_properties(0).multi_processor_count
        mhz = float(subprocess.run(["nvidia-smi", "--id=0", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits"],
                                   capture_output=True, text=True).stdout.strip() or 0)
        for bits in (2, 3, 4, 5, 6):
            w = ctx.prepare(synthetic.make_layer(1024, 1024, bits, seed=synthetic.BASE_SEED + 900 + bits))
            clk = w.decode_rate(400)
            out[f"K{bits}"] = {"clocks_per_tile_per_subpartition": round(clk, 1),
                               "GBps_ceiling_at_max_clock": round(4 * sm * mhz * 1e6 / clk * 32 * bits / 1e9, 0)}
            if bits == 4:  # how much of it is latency that more warps would hide
                out["K4_warps_per_sm"] = {str(n): round(w.decode_rate(400, warps_per_sm=n), 1) for n in (8, 16, 32)}
            w.close()
        out["sm_max_mhz"] = mhz
        out["status"] = ctx.device_status()
        print(json.dumps(out))
    elif args.case == "gemm":
        print(json.dumps({"case": "gemm 4096->12288 K4", **gemm_case(torch, ctx, stream, [2048], reps=2),
                          "status": ctx.device_status()}))
    elif args.case == "gemm-small":
        print(json.dumps({"case": "gemm 4096->12288 K4, one row tile with K partitions",
                          **gemm_case(torch, ctx, stream, [128], reps=2), "status": ctx.device_status()}))
    else:
        print(json.dumps({"case": "moe bank 32, top-8, 4096/2048 K2", **moe_case(torch, ctx, stream, [8], reps=2),
                          "status": ctx.device_status()}))


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from strix_trellis_b200 import native as N, synthetic
    from strix_trellis_b200.runtime import Context

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = Context(local)

    # ---- weights: the same number of device copies of every shape; one step launches each
    # copy once, shape after shape, so a copy is read again only after the other 1.2 GB
    # (ten times L2) went through ---------------------------------------------------------
    clones = CLONES
    groups, total_bytes, launches = [], 0, 0
    for k, (inputs, outputs) in enumerate(SHAPES):
        layer = synthetic.make_layer(inputs, outputs, BITS, seed=synthetic.BASE_SEED + k)
        ws = [ctx.prepare(layer) for _ in range(clones)]
        x = torch.from_numpy(synthetic.make_activations(ROWS, inputs, seed=synthetic.BASE_SEED + 50 + k)).cuda()
        y = torch.empty((ROWS, outputs), dtype=torch.float32, device="cuda")
        groups.append(dict(layer=layer, weights=ws, x=x, y=y, hx=x.cpu().pin_memory(),
                           hy=torch.empty((ROWS, outputs)).pin_memory()))
        total_bytes += clones * layer.packed_bytes
        launches += clones

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for g in groups:
            g["plans"] = [w.plan(g["x"], g["y"], N.OP_GEMV, stream=stream) for w in g["weights"]]
        for g in groups:  # correctness before timing: first clone against the CPU contract
            g["plans"][0].submit()
        stream.synchronize()
    from oracle import c_oracle
    for g in groups:
        layer = g["layer"]
        want = c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, BITS, 2, g["x"].cpu().numpy())
        err = np.abs(g["y"].cpu().numpy() - want).max()
        if not err <= 5e-4 * max(1.0, np.abs(want).max()):
            raise SystemExit(f"output check failed before timing: maxabs {err}")

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for g in groups:
                for p in g["plans"]:
                    p.submit()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput: `value` -------------------------------------------
    clocks = ClockSampler(local).__enter__()  # samples through the timed regions below
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        # keep the GPU under the same load until the sampler has a few readings
        t_end = time.time() + 0.6
        while time.time() < t_end:
            graph.replay()
        stream.synchronize()
    # per-shape launch time: the shape's copies as one graph, L2 flushed (256 MB written)
    # before each timed replay because the smallest shape's copies alone would fit in L2
    per_shape = {}
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    with torch.cuda.stream(stream):
        for g in groups:
            sub = torch.cuda.CUDAGraph()
            with torch.cuda.graph(sub, stream=stream):
                for p in g["plans"]:
                    p.submit()
            sub.replay()
            stream.synchronize()
            total_ms = 0.0
            for _ in range(3):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                sub.replay()
                b.record(stream)
                stream.synchronize()
                total_ms += a.elapsed_time(b)
            us = total_ms * 1e3 / 3 / len(g["plans"])
            layer = g["layer"]
            per_shape[f"{layer.inputs}x{layer.outputs}"] = {
                "us_per_launch": round(us, 3), "GBps": round(layer.packed_bytes / us / 1e3, 1)}
            del sub
    del flush
    ms_t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms = float(ms_t.item())
    ms_per_step = ms / args.steps
    value = world * total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: host activations in, host outputs out ---------------------------------
    # The step's 96 activation rows sit in ONE pinned host buffer and its 96 output rows return
    # to ONE pinned host buffer: [copies in, 96 x strix_linear_plan_submit, copies out] is the
    # timed unit (captured once, replayed), every call reading its own slice and writing its own.
    e2e_steps = max(1, min(args.steps, 10))
    n_in = sum(len(g["weights"]) * g["layer"].inputs for g in groups) * ROWS
    n_out = sum(len(g["weights"]) * g["layer"].outputs for g in groups) * ROWS
    hx_all, hy_all = torch.empty(n_in).pin_memory(), torch.empty(n_out).pin_memory()
    dx_all = torch.empty(n_in, dtype=torch.float32, device="cuda")
    dy_all = torch.empty(n_out, dtype=torch.float32, device="cuda")
    # launches whose rows travel in one copy each way: a whole shape (chunks of six measured
    # slower: every chunk boundary breaks the chain of programmatic launches)
    E2E_CHUNK = CLONES
    e2e_plans, spans, oi, oo = [], [], 0, 0  # spans: per chunk of one shape (plans, input slice, output slice)
    with torch.cuda.stream(stream):
        for g in groups:
            i_n, o_n = g["layer"].inputs * ROWS, g["layer"].outputs * ROWS
            for c0 in range(0, len(g["weights"]), E2E_CHUNK):
                i0, o0, first = oi, oo, len(e2e_plans)
                for w in g["weights"][c0:c0 + E2E_CHUNK]:
                    hx_all[oi:oi + i_n] = g["hx"].reshape(-1)
                    e2e_plans.append(w.plan(dx_all[oi:oi + i_n].view(ROWS, -1), dy_all[oo:oo + o_n].view(ROWS, -1),
                                            N.OP_GEMV, stream=stream))
                    oi, oo = oi + i_n, oo + o_n
                spans.append((e2e_plans[first:], slice(i0, oi), slice(o0, oo)))
    # the widest outputs first: what is still on its way back when the last launch ends is small
    spans.sort(key=lambda sp: -(sp[2].stop - sp[2].start))
    h2d, d2h = n_in * 4, n_out * 4
    # Copies are pipelined by chunk on a second stream (fork / join inside the capture): the
    # rows of chunk k+1 come in and the rows of chunk k-1 go out while chunk k computes.
    copy_stream = torch.cuda.Stream()
    e2e_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(e2e_graph, stream=stream):
            ready = []
            copy_stream.wait_stream(stream)  # fork
            with torch.cuda.stream(copy_stream):
                for _, xs, _ in spans:
                    dx_all[xs].copy_(hx_all[xs], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                    ready.append(ev)
            done = []
            for (plans, _, _), ev in zip(spans, ready):
                stream.wait_event(ev)
                for p in plans:
                    p.submit()
                ev2 = torch.cuda.Event()
                ev2.record(stream)
                done.append(ev2)
            with torch.cuda.stream(copy_stream):
                for (_, _, ys), ev2 in zip(spans, done):
                    copy_stream.wait_event(ev2)
                    hy_all[ys].copy_(dy_all[ys], non_blocking=True)
            stream.wait_stream(copy_stream)  # join
        for _ in range(3):
            e2e_graph.replay()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(e2e_steps):
            e2e_graph.replay()
        b.record(stream)
        barrier()
        e2e_ms = a.elapsed_time(b) / e2e_steps
    # the rows that came back are the rows the resident run produced (same weights, same input)
    oo = 0
    for g in groups:
        o_n = g["layer"].outputs * ROWS
        for _ in g["weights"]:
            if not torch.equal(hy_all[oo:oo + o_n], g["y"].cpu().reshape(-1)):
                raise SystemExit("end-to-end output row differs from the device-resident row")
            oo += o_n
    for p in e2e_plans:
        p.close()
    e2e_t = torch.tensor([e2e_ms], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_value = world * total_bytes / (float(e2e_t.item()) * 1e-3) / 1e9

    clocks.__exit__()
    clock_summary = clocks.summary()

    # ---- the same step as two and four independent chains of launches on as many streams ----
    # Reported beside the headline, not as it: a launch of the headline chain starts when the
    # one before it has ended; here copy i runs on chain i % chains, so one chain's launch
    # decodes while another chain's launch is in its fold tail -- what a caller with
    # independent projections (q/k/v, gate/up, experts) gets.
    two_chains = None
    if not args.no_extra and rank == 0:
        two_chains = {}
        for chains in (2, 4):
            side = [torch.cuda.Stream() for _ in range(chains - 1)]
            for g in groups:
                g["y_side"], g["plans_side"] = [], {}
                for k, st2 in enumerate(side):
                    with torch.cuda.stream(st2):
                        yb = torch.zeros_like(g["y"])
                        g["y_side"].append(yb)
                        for i in range(k + 1, len(g["weights"]), chains):  # copy i runs on chain i % chains
                            g["plans_side"][i] = g["weights"][i].plan(g["x"], yb, N.OP_GEMV, stream=st2)
                        st2.synchronize()
            multi = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(multi, stream=stream):
                    for st2 in side:
                        st2.wait_stream(stream)  # fork
                    for g in groups:
                        for i in range(len(g["weights"])):
                            (g["plans"][i] if i % chains == 0 else g["plans_side"][i]).submit()
                    for st2 in side:
                        stream.wait_stream(st2)  # join
                for _ in range(3):
                    multi.replay()
                stream.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(args.steps):
                    multi.replay()
                b.record(stream)
                stream.synchronize()
                multi_ms = a.elapsed_time(b) / args.steps
            for g in groups:
                for yb in g["y_side"]:
                    if not torch.equal(yb, g["y"]):
                        raise SystemExit("multi-chain run: output row differs from the single-chain row")
                for q in g["plans_side"].values():
                    q.close()
                g["y_side"], g["plans_side"] = [], {}
            two_chains[f"chains{chains}"] = {"GBps": round(total_bytes / (multi_ms * 1e-3) / 1e9, 1),
                                             "ms_per_step": round(multi_ms, 4)}
            del multi

    # ---- the other configurations of the metric, outside the timed region above ----------
    for g in groups:  # free the clone rotations first
        for p in g["plans"]:
            p.close()
        for w in g["weights"]:
            w.close()
    extra = {}
    if not args.no_extra:
        gemm_peak = 2250.0
        if (ROOT / "MEASURED_PEAKS.json").exists():
            gemm_peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
        if rank == 0:
            extra["gemv_sweep_independent_chains"] = two_chains
            gemm = gemm_case(torch, ctx, stream, [128, 512, 2048, 8192])
            for v in gemm.values():
                v["frac_of_measured_dense_peak"] = round(v["TFLOPs"] / gemm_peak, 3)
            extra["gemv_4096x14336_rates_rows"] = gemv_sweep(torch, ctx, stream)
            extra["prefill_gemm_K4_4096x12288"] = gemm
            for bits in (5, 6):
                other = gemm_case(torch, ctx, stream, [2048, 8192], bits=bits)
                for v in other.values():
                    v["frac_of_measured_dense_peak"] = round(v["TFLOPs"] / gemm_peak, 3)
                extra[f"prefill_gemm_K{bits}_4096x12288"] = other
            extra["moe_bank32_top8_K2_one_rank"] = moe_case(torch, ctx, stream, [1, 8, 64])
        if world > 1:
            dist.barrier()
        extra_tp = tp_case(torch, dist, ctx, stream, rank, world)
        extra_ep = ep_case(torch, dist, ctx, stream, rank, world)
        if rank == 0:
            extra[f"tp_dense_K5_world{world}"] = extra_tp
            extra[f"moe_256experts_top8_K2_world{world}"] = extra_ep
    status = ctx.device_status()
    if status:
        raise SystemExit(f"device status word {status:#x}: a bounded wait gave up; numbers invalid")

    if rank == 0:
        peak, peak_kind = measured_peak()
        avg_launch_us = ms_per_step * 1e3 / launches
        achieved = total_bytes / launches / avg_launch_us / 1e3  # GB/s per launch, one GPU
        traffic = None
        # DRAM bytes per packed weight byte of this kernel, from the committed ncu summary of
        # the 4096x14336 case; traffic grows in proportion to the packed bytes of a launch
        tpath = ROOT / "profiles" / "gemv_row_k4_4096x14336.md"
        if tpath.exists():
            for text in tpath.read_text().splitlines():
                if text.strip().startswith("dram_bytes_per_packed_byte"):
                    traffic = float(text.split("=")[1])
        base, _ = cpu_baseline() if world == 1 else (None, None)
        if base is not None:
            base["numpy_reference"] = numpy_baseline()
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 weights, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "bits": BITS, "rows": ROWS,
                       "cold_weights": f"{CLONES} device copies per shape, each launched once per step: 1.28 GB (10x L2) between two reads of a copy",
                       "launches_per_step": launches, "parallelism": f"replicas x{world}",
                       "per_shape": per_shape},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_kind": peak_kind,
                         "traffic": None if traffic is None else round(traffic * total_bytes / launches),
                         "kernel": "gemv_row_kernel<4, mul1>",
                         "algorithmic_bytes_per_launch": round(total_bytes / launches)},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "gpu_launches": launches * args.steps,
            "clocks": clock_summary,
            "extra": extra,
        }
        if base is not None:
            line["cpu_baseline"] = base
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the GEMM / MoE / TP side measurements")
    ap.add_argument("--case", choices=["gemv", "gemm", "gemm-small", "moe", "decode"], help="run one small profiling workload and exit")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
