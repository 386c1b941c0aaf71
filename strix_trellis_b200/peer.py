"""Exchange arenas of the ranks of one node (strix_b200_peer_*): creation, hand-over of the
64-byte handles through torch.distributed's object collectives (host side, once), and typed
wrappers of the three exchange kernels.  torch tensors only carry device pointers here.

A group belongs to ONE layer: all ranks must issue the same sequence of exchanges on it, and a
layer that runs an even number of exchanges per step finds every payload at a fixed address
(the parity of an exchange is its running number modulo two)."""
import ctypes as C

import torch

from . import native as N
from .runtime import _cur_stream


class _Raw:
    """Device memory as an array-interface object, so that torch can alias it."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerGroup:
    def __init__(self, ctx, arena_bytes, rank=0, world=1, group=None, local_ranks=1):
        """One arena per local rank (`local_ranks` = 1 in production; = world when every rank is
        played by this process on this device, which is how the protocol is tested on one GPU)."""
        if not 1 <= world <= N.PEER_RANKS or not 1 <= local_ranks <= world or rank + local_ranks > world:
            raise ValueError("bad rank layout")
        self.ctx, self.lib = ctx, ctx.lib
        self.rank, self.world, self.local = rank, world, local_ranks
        self.arena_bytes = int(arena_bytes + N.PEER_CONTROL_BYTES + 255) // 256 * 256
        self.cursor = N.PEER_CONTROL_BYTES
        self.arenas, handles = [], []
        for _ in range(local_ranks):
            ptr, handle = N.vp(), C.create_string_buffer(N.PEER_HANDLE_BYTES)
            N.check(self.lib.strix_b200_peer_arena_create(ctx.handle, self.arena_bytes, C.byref(ptr), handle),
                    "strix_b200_peer_arena_create")
            self.arenas.append(ptr.value)
            handles.append(handle.raw)
        table = None
        if local_ranks < world:
            import torch.distributed as dist
            every = [None] * world
            dist.all_gather_object(every, handles[0], group=group)
            table = C.create_string_buffer(b"".join(every), world * N.PEER_HANDLE_BYTES)
        local = (N.vp * local_ranks)(*self.arenas)
        self.handle = N.vp()
        N.check(self.lib.strix_b200_peer_group_create(ctx.handle, local, local_ranks, rank, self.arena_bytes, table,
                                                      world, C.byref(self.handle)), "strix_b200_peer_group_create")
        if local_ranks < world:
            import torch.distributed as dist
            dist.barrier(group=group)  # nobody stores into an arena before everybody has mapped it

    def set_wait_polls(self, polls):
        """How long a wait for a peer polls before it reports bit 5 of the device status word."""
        N.check(self.lib.strix_b200_peer_group_set_wait_polls(self.handle, int(polls)),
                "strix_b200_peer_group_set_wait_polls")

    # -- regions --------------------------------------------------------------------------
    def reserve(self, payload_bytes):
        """Offset of a fresh region for an exchange whose payload is `payload_bytes`."""
        at = self.cursor
        self.cursor = (at + 2 * payload_bytes + 255) // 256 * 256
        if self.cursor > self.arena_bytes:
            raise ValueError("arena too small for this layer's regions")
        return at

    def view(self, local_index, offset, shape, dtype=torch.float32):
        """Arena memory of local rank `local_index` as a tensor (no copy)."""
        count = 1
        for d in shape:
            count *= d
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        raw = torch.as_tensor(_Raw(self.arenas[local_index] + offset, nbytes), device="cuda")
        return raw.view(dtype).view(*shape)

    # -- exchanges ------------------------------------------------------------------------
    def sum_rows(self, rows, region, stream=None):
        """rows: one contiguous float32 tensor per local rank, replaced by the sum over ranks."""
        ptrs = (N.vp * self.local)(*[t.data_ptr() for t in rows])
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_peer_sum(self.handle, ptrs, rows[0].numel(), region, C.byref(sd)),
                "strix_b200_peer_sum")

    def gather(self, rows, row_at, matrices, stream=None, tagged=False):
        """matrices: up to three dicts with `blocks` (one tensor of 32-bit words per local rank),
        `results` (same, or None), `widths`, `col_at` (per rank), `total_cols`, `region`.
        `tagged`: every word travels with the exchange number (no fence, no flag step); needs
        results, even widths and a region for 8 bytes per word."""
        d = N.PeerGatherDesc()
        d.struct_size, d.abi_version, d.matrices = C.sizeof(d), N.ABI_VERSION, len(matrices)
        d.flags = N.PEER_GATHER_TAGGED if tagged else 0
        for r in range(self.world):
            d.rows[r], d.row_at[r] = rows[r], row_at[r]
        for m, spec in enumerate(matrices):
            mx = d.matrix[m]
            mx.total_cols, mx.region = spec["total_cols"], spec["region"]
            for r in range(self.world):
                mx.width[r], mx.col_at[r] = spec["widths"][r], spec["col_at"][r]
            for i in range(self.local):
                mx.block[i] = spec["blocks"][i].data_ptr()
                res = spec.get("results")
                mx.result[i] = res[i].data_ptr() if res is not None and res[i] is not None else None
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_peer_gather(self.handle, C.byref(d), C.byref(sd)), "strix_b200_peer_gather")

    def return_routes(self, each, ids, row_valid, first_expert, experts, tokens, tokens_per_rank, top_k, width,
                      region, stream=None):
        """each / ids / row_valid / first_expert / experts: one entry per local rank (device
        pointers as ints for the first three)."""
        d = N.PeerReturnDesc()
        d.struct_size, d.abi_version = C.sizeof(d), N.ABI_VERSION
        for i in range(self.local):
            d.each[i], d.ids[i], d.row_valid[i] = each[i], ids[i], row_valid[i]
            d.first_expert[i], d.experts[i] = first_expert[i], experts[i]
        d.tokens, d.tokens_per_rank, d.top_k, d.width, d.region = tokens, tokens_per_rank, top_k, width, region
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_peer_return_routes(self.handle, C.byref(d), C.byref(sd)),
                "strix_b200_peer_return_routes")

    def close(self):
        if self.handle:
            torch.cuda.synchronize()
            if self.local < self.world:
                import torch.distributed as dist
                if dist.is_initialized():
                    dist.barrier()  # nobody unmaps while a peer may still store
            N.check(self.lib.strix_b200_peer_group_destroy(self.handle), "strix_b200_peer_group_destroy")
            self.handle = N.vp()
            for a in self.arenas:
                N.check(self.lib.strix_b200_peer_arena_destroy(self.ctx.handle, a), "strix_b200_peer_arena_destroy")
            self.arenas = []
