"""Load-time tensor-parallel partitions of EXL3 groups for any number of ranks, and the
collectives that recombine per-rank results.

Generalises the reference's two-rank, fixed-geometry helper (python/strix_trellis/tp.py:
55-83) to N ranks and any H128-aligned geometry.  Compressed weights are never expanded:
an output (column) partition repacks its tile stride once at export, an input (row)
partition borrows contiguous storage.  The math contract is the reference's
(docs/TP_RANK.md:150-156): column shards are concatenated in rank order, row shards are
summed with the bias on exactly one rank, replicas are not summed.
"""
import numpy as np

AXES = ("output", "input", "replicate")


def h128_bounds(total, parts):
    """`parts` contiguous H128-aligned ranges covering [0, total); the first
    (total/128) % parts ranges are one block longer."""
    if total % 128 or parts < 1 or total // 128 < parts:
        raise ValueError("need at least one H128 block per rank")
    base, extra = divmod(total // 128, parts)
    out, begin = [], 0
    for r in range(parts):
        size = base + (1 if r < extra else 0)
        out.append((begin * 128, (begin + size) * 128))
        begin += size
    return out


def rank_partition(tensor, axis, rank, world, *, bias_rank=0):
    """The shard of `tensor` (container.Exl3Tensor or anything with the same slicing
    methods) that rank `rank` of `world` owns along `axis`."""
    if axis not in AXES:
        raise ValueError("axis must be 'output', 'input' or 'replicate'")
    if type(rank) is not int or type(world) is not int or not 0 <= rank < world:
        raise ValueError("rank must be an integer in [0, world)")
    if type(bias_rank) is not int or not 0 <= bias_rank < world:
        raise ValueError("bias_rank must be an integer in [0, world)")
    if axis == "replicate":
        return tensor
    if axis == "output":
        b0, b1 = h128_bounds(tensor.output_size, world)[rank]
        return tensor.slice_outputs(b0, b1)
    a0, a1 = h128_bounds(tensor.input_size, world)[rank]
    return tensor.slice_inputs(a0, a1, include_bias=rank == bias_rank)


def expert_owner(expert_id, experts, world):
    """Contiguous expert ownership: expert e lives on rank e // ceil(experts/world)."""
    per = -(-experts // world)
    return expert_id // per


# ---- the shard-boundary steps as library collectives ------------------------------------------
# For callers that own the exchange themselves (the reference's model) and for the host-side
# tests, which run them over gloo.  The GPU layers in tp_runtime.py do not use these: their
# exchange is a kernel that stores into the peers' memory (peer.py).
def all_reduce_rows(local, group=None):
    """Row-parallel (input-split) recombination: sum of rank outputs, in place."""
    import torch.distributed as dist
    dist.all_reduce(local, op=dist.ReduceOp.SUM, group=group)
    return local


_COLUMN_INDEX = {}


def all_gather_columns(local, widths, group=None):
    """Column-parallel recombination: rank r's [rows, widths[r]] block lands at its column
    offset of the [rows, sum(widths)] result.  Shards may be uneven (e.g. 1010 H128 blocks
    over 4 or 8 ranks): every rank pads to the widest shard for the collective, and one
    gather with a cached column index drops the padding afterwards."""
    import torch
    import torch.distributed as dist
    world = len(widths)
    rows, wmax = local.shape[0], max(widths)
    padded = local if local.shape[1] == wmax else torch.nn.functional.pad(local, (0, wmax - local.shape[1]))
    gathered = torch.empty((world * rows, wmax), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered, padded.contiguous(), group=group)
    by_row = gathered.view(world, rows, wmax).permute(1, 0, 2).reshape(rows, world * wmax)
    if min(widths) == wmax:
        return by_row
    key = (tuple(widths), str(local.device))
    index = _COLUMN_INDEX.get(key)
    if index is None:
        index = torch.cat([torch.arange(r * wmax, r * wmax + widths[r]) for r in range(world)]).to(local.device)
        _COLUMN_INDEX[key] = index
    return by_row.index_select(1, index)
