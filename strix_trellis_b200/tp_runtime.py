"""Tensor- and expert-parallel layers over the per-rank C ABI: every rank runs the complete
local operator on its shard (one process per GPU) and the ranks meet only at the shard
boundary, through peer memory over NVLink (strix_b200_peer_*, one kernel per exchange, no
library collective on the forward path).  Math contract of the reference
(docs/TP_RANK.md:150-156): row-parallel outputs are summed, column-parallel outputs are
concatenated in rank order, the bias lives on exactly one rank, expert outputs are combined at
the token's home rank in ascending slot order.

Every forward is a fixed sequence of kernel launches on the caller's current stream: no host
synchronisation, no allocation after the first call, capturable into a CUDA graph on any number
of ranks.  A plan is frozen for the stream it was first used on; using a layer from another
stream builds another plan (plans are cached per stream and buffer set).
"""
import numpy as np
import torch

from . import tp
from .peer import PeerGroup
from .runtime import DensePlan, MoePlan, _cur_stream
from . import native as N
import ctypes as C


def _stream_key():
    return torch.cuda.current_stream().cuda_stream


class RowParallelLinear:
    """Input (split-K) partition: rank r multiplies its slice of x by its K slice of the
    weights; the [rows, N] partial outputs are summed over the ranks in rank order."""

    def __init__(self, ctx, tensor, rank, world, group=None, bias_rank=0, full_inputs=None, max_rows=8):
        """`tensor` is the whole layer, or (with `full_inputs` = the layer's input size) this
        rank's shard already cut, e.g. by a loader that reads only its own slice."""
        self.rank, self.world = rank, world
        self.bounds = tp.h128_bounds(full_inputs or tensor.input_size, world)
        shard = tensor if full_inputs else tp.rank_partition(tensor, "input", rank, world, bias_rank=bias_rank)
        a0, a1 = self.bounds[rank]
        if shard.input_size != a1 - a0:
            raise ValueError("shard does not match this rank's input range")
        self.weights = ctx.prepare(shard)
        self.plans = {}
        self.ctx, self.group, self.peers = ctx, group, None
        self.max_rows = max_rows

    def _exchange(self):
        """The exchange arena, set up (collectively: every rank must get here) at the first
        forward; `local` alone never needs it."""
        if self.peers is None:
            payload = self.world * self.max_rows * self.weights.outputs * 8  # every value travels with its arrival mark
            self.peers = PeerGroup(self.ctx, 2 * payload + 4096, self.rank, self.world, self.group)
            self.region = self.peers.reserve(payload)
        return self.peers

    def local(self, x_full, y=None):
        """y = Linear_r(x_full[:, a0:a1]) on the strided column view, no copy.  Plans are
        frozen per (stream, activation buffer, output buffer) and reused."""
        a0, a1 = self.bounds[self.rank]
        if y is None:
            y = torch.empty((x_full.shape[0], self.weights.outputs), dtype=torch.float32, device=x_full.device)
        key = (_stream_key(), x_full.data_ptr(), tuple(x_full.shape), x_full.stride(0), y.data_ptr(), y.stride(0))
        plan = self.plans.get(key)
        if plan is None:
            plan = self.plans[key] = DensePlan(self.weights, x_full[:, a0:a1], y)
        plan.submit()
        return y

    def forward(self, x_full, y=None):
        y = self.local(x_full, y)
        if self.world > 1:
            if y.shape[0] > self.max_rows or not y.is_contiguous():
                raise ValueError("row count beyond the exchange region this layer reserved")
            self._exchange().sum_rows([y], self.region)
        return y

    def close(self):
        for plan in self.plans.values():
            plan.close()
        self.plans.clear()
        if self.peers:
            self.peers.close()
        self.weights.close()


class ColumnParallelLinear:
    """Output partition (LM head): rank r owns an H128-aligned column range; every rank's block
    of logits is stored into every rank's result at its column offset (uneven shards need no
    padding)."""

    # logits of one call up to this many bytes travel as tagged words (twice the bytes, but no
    # fence and no flag step: measured 83 against 90 us for one row of 129280 logits on two GPUs,
    # and 123 against 112 us for eight rows, where the doubled traffic costs more)
    TAGGED_LIMIT = 1 << 20

    def __init__(self, ctx, tensor, rank, world, group=None, full_outputs=None, max_rows=8):
        self.rank, self.world = rank, world
        self.bounds = tp.h128_bounds(full_outputs or tensor.output_size, world)
        self.widths = [b - a for a, b in self.bounds]
        self.total = self.bounds[-1][1]
        shard = tensor if full_outputs else tp.rank_partition(tensor, "output", rank, world)
        if shard.output_size != self.widths[rank]:
            raise ValueError("shard does not match this rank's output range")
        self.weights = ctx.prepare(shard)
        self.plans, self.blocks, self.results = {}, {}, {}
        self.ctx, self.group, self.peers = ctx, group, None
        self.max_rows = max_rows

    def _exchange(self):
        """The exchange arena, set up (collectively: every rank must get here) at the first
        forward; `local` alone never needs it."""
        if self.peers is None:
            # few rows travel as tagged words (8 bytes per logit, lowest latency), more rows plainly
            plain = self.max_rows * self.total * 4
            payload = max(plain, 2 * min(plain, self.TAGGED_LIMIT))
            self.peers = PeerGroup(self.ctx, 2 * payload + 4096, self.rank, self.world, self.group)
            self.region = self.peers.reserve(payload)
        return self.peers

    def local(self, x, y=None):
        """This rank's logits block; plans are frozen per (stream, activation, output) buffers."""
        if y is None:
            y = self.blocks.get((x.shape[0], x.device))
            if y is None:
                y = self.blocks[(x.shape[0], x.device)] = torch.empty(
                    (x.shape[0], self.weights.outputs), dtype=torch.float32, device=x.device)
        key = (_stream_key(), x.data_ptr(), tuple(x.shape), x.stride(0), y.data_ptr(), y.stride(0))
        plan = self.plans.get(key)
        if plan is None:
            plan = self.plans[key] = DensePlan(self.weights, x, y)
        plan.submit()
        return y

    def forward(self, x):
        """[rows, full outputs] logits; the tensor is reused by the next forward of the same row
        count."""
        y = self.local(x)
        if self.world == 1:
            return y
        rows = x.shape[0]
        if rows > self.max_rows:
            raise ValueError("row count beyond the exchange region this layer reserved")
        out = self.results.get(rows)
        if out is None:
            out = self.results[rows] = torch.empty((rows, self.total), dtype=torch.float32, device=x.device)
        self._exchange().gather([rows] * self.world, [0] * self.world,
                          [dict(blocks=[y], results=[out], widths=self.widths, col_at=[a for a, _ in self.bounds],
                                total_cols=self.total, region=self.region)],
                          tagged=rows * self.total * 4 <= self.TAGGED_LIMIT)
        return out

    def close(self):
        for plan in self.plans.values():
            plan.close()
        self.plans.clear()
        if self.peers:
            self.peers.close()
        self.weights.close()


class ExpertParallelMoE:
    """Experts owned contiguously (expert e on rank e // ceil(E/world)); tokens live rank-major
    (`max_tokens` slots per rank).  A step:

      1. every rank's token rows, route ids and scores are stored into every rank (one
         exchange): all ranks see all routes and apply the same row rules, so they agree on
         which rows are valid without talking about it;
      2. a device-routed plan whose bank is this rank's window of the expert ids runs routing,
         gate/up, SwiGLU and down for the routes this rank owns (an expert's weights are read
         once per eight rows routed to it, whoever sent them);
      3. each owner stores the output row of route (t, s) into the home rank of token t (second
         exchange);
      4. the home rank combines its tokens' rows in ascending slot order from +0, a zero score
         skips its slot, an invalid route row becomes NaN -- bit for bit what the single-rank
         plan does, which a sum across ranks would not give.

    Two exchanges per step keep every payload at a fixed address, so the step is five kernels
    and two exchanges on one stream with nothing on the host in between."""

    PAD = 0xFFFFFFFF  # route id of an empty token slot: invalid on every rank, runs nothing

    def __init__(self, ctx, local_experts, experts_total, rank, world, model, max_tokens, top_k, group=None):
        self.ctx, self.rank, self.world = ctx, rank, world
        self.per_rank = -(-experts_total // world)
        self.first = rank * self.per_rank
        if len(local_experts) != min(self.per_rank, experts_total - self.first):
            raise ValueError("this rank owns a different number of experts")
        self.model, self.top_k, self.slots = model, top_k, max_tokens
        self.tokens_all = world * max_tokens
        f32 = dict(dtype=torch.float32, device="cuda")
        self.x_in = torch.zeros((max_tokens, model), **f32)
        self.ids_in = torch.full((max_tokens, top_k), self.PAD - (1 << 32), dtype=torch.int32, device="cuda")
        self.sc_in = torch.zeros((max_tokens, top_k), **f32)
        self.y = torch.zeros((max_tokens, model), **f32)
        self.peers = None
        if world == 1:
            x_all, ids_all, sc_all = self.x_in, self.ids_in, self.sc_in
        else:
            # Few tokens: the gather carries tagged words (8 bytes per word, no fence and no flag
            # step) into tensors of this layer; many tokens: plain words that the plan reads where
            # they land in the arena.
            self.tagged = (self.tokens_all * model * 4 <= ColumnParallelLinear.TAGGED_LIMIT and model % 2 == 0
                           and top_k % 2 == 0)
            word = 8 if self.tagged else 4
            sizes = [self.tokens_all * model * word, self.tokens_all * top_k * word, self.tokens_all * top_k * word,
                     max_tokens * top_k * model * 4]
            self.peers = PeerGroup(ctx, 2 * sum(sizes) + 8192, rank, world, group)
            self.regions = [self.peers.reserve(n) for n in sizes]
            if self.tagged:
                x_all = torch.zeros((self.tokens_all, model), **f32)
                ids_all = torch.zeros((self.tokens_all, top_k), dtype=torch.int32, device="cuda")
                sc_all = torch.zeros((self.tokens_all, top_k), **f32)
                self.gathered = [x_all, ids_all, sc_all]
            else:
                # the gather is this group's exchange 1, 3, 5, ... (parity 1), the return 2, 4, ... (parity 0)
                x_all = self.peers.view(0, self.regions[0] + sizes[0], (self.tokens_all, model))
                ids_all = self.peers.view(0, self.regions[1] + sizes[1], (self.tokens_all, top_k), torch.int32)
                sc_all = self.peers.view(0, self.regions[2] + sizes[2], (self.tokens_all, top_k))
                self.gathered = [None, None, None]
            self.back = self.peers.view(0, self.regions[3], (max_tokens, top_k, model))
        self.ids_all = ids_all
        self.sink = torch.zeros((self.tokens_all, model), **f32)  # the plan's own (unused) output
        self.plan = MoePlan(ctx, local_experts, x_all, self.sink, ids_all, sc_all, device_routed=True)
        N.check(ctx.lib.strix_b200_moe_plan_set_window(self.plan.handle, self.first, experts_total), "set_window")
        each, valid = N.vp(), N.vp()
        N.check(ctx.lib.strix_b200_moe_plan_rows(self.plan.handle, C.byref(each), C.byref(valid)), "plan_rows")
        self.each_ptr, self.valid_ptr = each.value, valid.value
        self.plan_stream = _stream_key()

    def stage(self, x, route_ids, route_scores):
        """Copies one step's inputs into the layer's static buffers (device copies on the current
        stream).  x [T, model] float32; route_ids [T, top_k] global expert ids; T <= max_tokens."""
        x = torch.as_tensor(x, device="cuda")
        tokens = x.shape[0]
        ids = torch.as_tensor(np.asarray(route_ids) if not torch.is_tensor(route_ids) else route_ids, device="cuda")
        scores = torch.as_tensor(np.asarray(route_scores, dtype=np.float32) if not torch.is_tensor(route_scores)
                                 else route_scores, device="cuda")
        if tokens > self.slots or tuple(ids.shape) != (tokens, self.top_k):
            raise ValueError("routes exceed the capacity this layer was created for")
        self.x_in[:tokens].copy_(x, non_blocking=True)
        self.ids_in[:tokens].copy_(ids.to(torch.int64).bitwise_and(0xFFFFFFFF).to(torch.int32) if ids.dtype != torch.int32
                                   else ids, non_blocking=True)
        self.ids_in[tokens:].fill_(self.PAD - (1 << 32))
        self.sc_in[:tokens].copy_(scores.to(torch.float32), non_blocking=True)
        return tokens

    def run(self, tokens, alpha=1.0):
        """One step on the staged inputs; returns y[:tokens] (a static buffer)."""
        if _stream_key() != self.plan_stream:
            raise RuntimeError("this layer's plan is frozen on the stream it was created on")
        ctx, lib = self.ctx, self.ctx.lib
        if self.world > 1:
            per, k = self.slots, self.top_k
            rows, row_at = [per] * self.world, [r * per for r in range(self.world)]
            one = lambda block, width, m: dict(blocks=[block], widths=[width] * self.world, col_at=[0] * self.world,
                                               total_cols=width, region=self.regions[m],
                                               results=[self.gathered[m]] if self.tagged else None)
            self.peers.gather(rows, row_at, [one(self.x_in, self.model, 0), one(self.ids_in, k, 1), one(self.sc_in, k, 2)],
                              tagged=self.tagged)
        N.check(lib.strix_b200_moe_plan_projections(self.plan.handle), "strix_b200_moe_plan_projections")
        if self.world > 1:
            self.peers.return_routes([self.each_ptr], [self.ids_all.data_ptr()], [self.valid_ptr], [self.first],
                                     [len(self.plan.keep[2])], self.tokens_all, self.slots, self.top_k, self.model,
                                     self.regions[3])
            rows_ptr = self.back.data_ptr()
        else:
            rows_ptr = self.each_ptr
        if tokens:
            sd = _cur_stream()
            N.check(lib.strix_b200_moe_combine_rows(ctx.handle, rows_ptr, self.sc_in.data_ptr(),
                                                    self.valid_ptr + 4 * self.rank * self.slots, tokens, self.top_k,
                                                    self.model, self.y.data_ptr(), self.model, alpha, 0.0, C.byref(sd)),
                    "strix_b200_moe_combine_rows")
        return self.y[:tokens]

    def forward(self, x, route_ids, route_scores, alpha=1.0):
        """x [T, model] float32; route_ids [T, top_k] (global expert ids) and route_scores
        [T, top_k] as CUDA tensors or host arrays; T <= max_tokens (T may be 0: the rank still
        takes part in both exchanges).  Returns y [T, model]."""
        return self.run(self.stage(x, route_ids, route_scores), alpha)

    def capture(self, tokens):
        """Freezes run() for `tokens` home tokens into a CUDA graph (any number of ranks: the step
        contains no library collective and nothing that allocates).  Returns
        run(x, ids, scores) -> y; y is a static buffer overwritten by the next run."""
        stream = torch.cuda.current_stream()
        self.run(tokens)  # every rank warms up the same number of steps: exchanges stay paired
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = self.run(tokens)

        def run(x, ids, scores):
            self.stage(x, ids, scores)
            graph.replay()
            return y
        self.graph = graph
        return run

    def close(self):
        self.graph = None
        self.plan.close()
        if self.peers:
            self.peers.close()
