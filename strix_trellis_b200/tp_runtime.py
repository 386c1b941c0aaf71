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
    (all-to-all) and combine at the token's home rank in ascending slot order from +0."""

    def __init__(self, ctx, local_experts, experts_total, rank, world, model, capacity, group=None):
        self.ctx, self.rank, self.world, self.group = ctx, rank, world, group
        self.per_rank = -(-experts_total // world)
        self.first = rank * self.per_rank
        self.model, self.capacity = model, capacity
        self.rows_in = torch.zeros((capacity, model), dtype=torch.float32, device="cuda")
        self.rows_out = torch.zeros((capacity, model), dtype=torch.float32, device="cuda")
        self.ids = torch.full((capacity,), 0x7FFFFFFF, dtype=torch.int32, device="cuda")  # invalid = idle slot
        self.ones = torch.ones((capacity,), dtype=torch.float32, device="cuda")
        self.plan = MoePlan(ctx, local_experts, self.rows_in, self.rows_out, self.ids, self.ones, device_routed=True)

    def forward(self, x, route_ids, route_scores, alpha=1.0):
        """x [T_home, model] CUDA; route_ids/scores [T_home, top_k] host arrays (global ids)."""
        import torch.distributed as dist
        tokens, top_k = route_ids.shape
        owner = route_ids // self.per_rank
        order = np.argsort(owner.ravel(), kind="stable")          # routes grouped by owner rank
        send_counts = np.bincount(owner.ravel(), minlength=self.world).astype(np.int64)
        send_rows = x[torch.from_numpy((order // top_k).astype(np.int64)).cuda()]
        send_ids = torch.from_numpy((route_ids.ravel()[order] % self.per_rank).astype(np.int32)).cuda()
        if self.world > 1:
            counts_t = torch.from_numpy(send_counts).cuda()
            recv_t = torch.empty_like(counts_t)
            dist.all_to_all_single(recv_t, counts_t, group=self.group)
            recv_counts = recv_t.cpu().numpy()
        else:
            recv_counts = send_counts
        n_recv = int(recv_counts.sum())
        if n_recv > self.capacity:
            raise ValueError("more routed rows than the plan's capacity")
        self.ids.fill_(0x7FFFFFFF)
        if self.world > 1:
            dist.all_to_all_single(self.rows_in[:n_recv], send_rows, recv_counts.tolist(), send_counts.tolist(),
                                   group=self.group)
            dist.all_to_all_single(self.ids[:n_recv], send_ids, recv_counts.tolist(), send_counts.tolist(),
                                   group=self.group)
        else:
            self.rows_in[:n_recv] = send_rows
            self.ids[:n_recv] = send_ids
        self.plan.submit()
        back = torch.empty((order.size, self.model), dtype=torch.float32, device="cuda")
        if self.world > 1:
            dist.all_to_all_single(back, self.rows_out[:n_recv], send_counts.tolist(), recv_counts.tolist(),
                                   group=self.group)
        else:
            back.copy_(self.rows_out[:n_recv])
        each = torch.empty((tokens * top_k, self.model), dtype=torch.float32, device="cuda")
        each[torch.from_numpy(order.astype(np.int64)).cuda()] = back
        each = each.view(tokens, top_k, self.model)
        scores = torch.from_numpy(np.ascontiguousarray(route_scores, dtype=np.float32)).cuda()
        y = torch.zeros((tokens, self.model), dtype=torch.float32, device="cuda")
        for s in range(top_k):  # ascending slot order; mul and add round separately
            term = scores[:, s:s + 1] * each[:, s]
            y = torch.where(scores[:, s:s + 1] == 0, y, y + term)
        return y * alpha if alpha != 1.0 else y

    def close(self):
        self.plan.close()
