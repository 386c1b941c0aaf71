"""Tensor- and expert-parallel layers over the per-rank C ABI: every rank runs the complete
local operator on its shard (one process per GPU) and torch.distributed (NCCL over NVLink)
runs only at the shard boundary.  Math contract of the reference (docs/TP_RANK.md:150-156):
row-parallel outputs are summed, column-parallel outputs are concatenated in rank order,
the bias lives on exactly one rank, expert outputs are combined at the token's home rank in
ascending slot order.  No kernel reads peer memory.
"""
import numpy as np
import torch

from . import tp
from .runtime import DensePlan, MoePlan


class RowParallelLinear:
    """Input (split-K) partition: rank r multiplies its slice of x by its K slice of the
    weights; all-reduce(sum) of the [rows, N] partial outputs."""

    def __init__(self, ctx, tensor, rank, world, group=None, bias_rank=0, full_inputs=None):
        """`tensor` is the whole layer, or (with `full_inputs` = the layer's input size) this
        rank's shard already cut, e.g. by a loader that reads only its own slice."""
        self.rank, self.world, self.group = rank, world, group
        self.bounds = tp.h128_bounds(full_inputs or tensor.input_size, world)
        shard = tensor if full_inputs else tp.rank_partition(tensor, "input", rank, world, bias_rank=bias_rank)
        a0, a1 = self.bounds[rank]
        if shard.input_size != a1 - a0:
            raise ValueError("shard does not match this rank's input range")
        self.weights = ctx.prepare(shard)
        self.plans = {}

    def local(self, x_full, y=None):
        """y = Linear_r(x_full[:, a0:a1]) on the strided column view, no copy.  Plans are
        frozen per (activation buffer, output buffer) pair and reused."""
        a0, a1 = self.bounds[self.rank]
        if y is None:
            y = torch.empty((x_full.shape[0], self.weights.outputs), dtype=torch.float32, device=x_full.device)
        key = (x_full.data_ptr(), tuple(x_full.shape), x_full.stride(0), y.data_ptr(), y.stride(0))
        plan = self.plans.get(key)
        if plan is None:
            plan = self.plans[key] = DensePlan(self.weights, x_full[:, a0:a1], y)
        plan.submit()
        return y

    def close(self):
        for plan in self.plans.values():
            plan.close()
        self.plans.clear()
        self.weights.close()

    def forward(self, x_full, y=None):
        y = self.local(x_full, y)
        if self.world > 1:
            tp.all_reduce_rows(y, self.group)
        return y


class ColumnParallelLinear:
    """Output partition (LM head): rank r owns an H128-aligned column range; all-gather of
    the logits (padded to the widest shard when the block count does not divide)."""

    def __init__(self, ctx, tensor, rank, world, group=None, full_outputs=None):
        self.rank, self.world, self.group = rank, world, group
        self.bounds = tp.h128_bounds(full_outputs or tensor.output_size, world)
        self.widths = [b - a for a, b in self.bounds]
        shard = tensor if full_outputs else tp.rank_partition(tensor, "output", rank, world)
        if shard.output_size != self.widths[rank]:
            raise ValueError("shard does not match this rank's output range")
        self.weights = ctx.prepare(shard)
        self.plans, self.outputs = {}, {}

    def local(self, x, y=None):
        """This rank's logits block; plans are frozen per (activation, output) buffer pair."""
        if y is None:
            y = self.outputs.get((x.shape[0], x.device))
            if y is None:
                y = self.outputs[(x.shape[0], x.device)] = torch.empty(
                    (x.shape[0], self.weights.outputs), dtype=torch.float32, device=x.device)
        key = (x.data_ptr(), tuple(x.shape), x.stride(0), y.data_ptr(), y.stride(0))
        plan = self.plans.get(key)
        if plan is None:
            plan = self.plans[key] = DensePlan(self.weights, x, y)
        plan.submit()
        return y

    def forward(self, x):
        y = self.local(x)
        return y if self.world == 1 else tp.all_gather_columns(y, self.widths, self.group)

    def close(self):
        for plan in self.plans.values():
            plan.close()
        self.plans.clear()
        self.weights.close()


class ExpertParallelMoE:
    """Experts owned contiguously (expert e on rank e // ceil(E/world)).  A step:
    dispatch every (token, slot) row to the owner of its expert (all-to-all), run the
    owner's experts on the received rows (a device-routed plan with one route per row and
    score 1, so a row's output IS down_e(SwiGLU(...)) bit for bit), return the rows
    (all-to-all) and combine at the token's home rank in ascending slot order from +0.

    The exchange uses a fixed capacity per rank pair (max_tokens * top_k rows, unused slots
    carry an invalid expert id and run nothing), so a step needs no host synchronisation:
    packing, the three collectives, the expert kernels and the combine are all enqueued."""

    INVALID = 0x7FFFFFFF

    def __init__(self, ctx, local_experts, experts_total, rank, world, model, max_tokens, top_k, group=None):
        self.ctx, self.rank, self.world, self.group = ctx, rank, world, group
        self.per_rank = -(-experts_total // world)
        self.model, self.top_k = model, top_k
        self.cap = max_tokens * top_k  # rows one rank can send to (or receive from) one rank
        rows = world * self.cap
        f32 = dict(dtype=torch.float32, device="cuda")
        self.send_x = torch.zeros((rows, model), **f32)
        self.recv_x = self.send_x if world == 1 else torch.zeros((rows, model), **f32)
        self.send_ids = torch.full((rows,), self.INVALID, dtype=torch.int32, device="cuda")
        self.recv_ids = self.send_ids if world == 1 else torch.full((rows,), self.INVALID, dtype=torch.int32, device="cuda")
        self.out_rows = torch.zeros((rows, model), **f32)
        self.back = self.out_rows if world == 1 else torch.zeros((rows, model), **f32)
        self.ones = torch.ones((rows,), **f32)
        self.rank_ids = torch.arange(world, device="cuda")
        self.plan = MoePlan(ctx, local_experts, self.recv_x, self.out_rows, self.recv_ids, self.ones, device_routed=True)
        self.graphs = []

    def forward(self, x, route_ids, route_scores, alpha=1.0):
        """x [T, model] CUDA float32; route_ids [T, top_k] (global expert ids) and route_scores
        [T, top_k] as CUDA tensors or host arrays; T <= max_tokens.  Returns y [T, model]."""
        import torch.distributed as dist
        ids = torch.as_tensor(np.asarray(route_ids) if not torch.is_tensor(route_ids) else route_ids).to("cuda").long()
        scores = torch.as_tensor(np.asarray(route_scores, dtype=np.float32) if not torch.is_tensor(route_scores)
                                 else route_scores).to("cuda", torch.float32)
        tokens, top_k = ids.shape
        if top_k != self.top_k or tokens * top_k > self.cap:
            raise ValueError("routes exceed the capacity this layer was created for")
        count = tokens * top_k
        flat = ids.reshape(-1)
        owner = flat // self.per_rank
        # slot of a route in the send buffer: its owner's section, then its rank among the routes
        # of this rank that go to the same owner, in route order (a running count per owner)
        mine = owner[:, None] == self.rank_ids[None, :]
        position = torch.cumsum(mine, 0).gather(1, owner[:, None]).squeeze(1) - 1
        slot = owner * self.cap + position
        self.send_ids.fill_(self.INVALID)
        self.send_ids[slot] = (flat - owner * self.per_rank).int()
        self.send_x[slot] = x.repeat_interleave(top_k, dim=0)
        if self.world > 1:
            dist.all_to_all_single(self.recv_x, self.send_x, group=self.group)
            dist.all_to_all_single(self.recv_ids, self.send_ids, group=self.group)
        self.plan.submit()
        if self.world > 1:
            dist.all_to_all_single(self.back, self.out_rows, group=self.group)
        each = self.back[slot] if count else self.back[:0]
        y = torch.empty((tokens, self.model), dtype=torch.float32, device="cuda")
        if tokens:  # ascending slot order from +0, a zero score skips its slot: the plan's own combine
            self.ctx.moe_combine(each.view(tokens, top_k, self.model), scores.contiguous(), y, alpha=alpha)
        return y

    def capture(self, tokens):
        """Freezes forward() for `tokens` home tokens into a CUDA graph over static input
        buffers.  Single-rank layers only: with the collectives inside the capture a two-rank
        run did not return, so multi-rank forwards stay eager.  Returns
        run(x, ids, scores) -> y; y is a static buffer overwritten by the next run."""
        if self.world != 1:
            raise ValueError("capture is offered for single-rank layers")
        x_in = torch.zeros((tokens, self.model), dtype=torch.float32, device="cuda")
        ids_in = torch.zeros((tokens, self.top_k), dtype=torch.long, device="cuda")
        sc_in = torch.zeros((tokens, self.top_k), dtype=torch.float32, device="cuda")
        stream = torch.cuda.current_stream()
        self.forward(x_in, ids_in, sc_in)  # warm-up outside the capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = self.forward(x_in, ids_in, sc_in)

        def run(x, ids, scores):
            x_in.copy_(x)
            ids_in.copy_(ids)
            sc_in.copy_(scores)
            graph.replay()
            return y
        self.graphs.append(graph)
        return run

    def close(self):
        self.graphs.clear()
        self.plan.close()
