"""Object layer over the C ABI.  torch tensors are used only as carriers of device
memory (data_ptr) and of the current CUDA stream; all arithmetic happens inside
libstrix_trellis.so."""
import ctypes as C

import numpy as np
import torch

from . import native as N


def _cur_stream(stream=None):
    if stream is None:
        stream = torch.cuda.current_stream()
    return N.stream_desc(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


class Context:
    """strix_context for one device (must be the calling thread's current device)."""

    def __init__(self, device=None):
        self.lib = N.load()
        if not torch.cuda.is_available():
            raise RuntimeError("strix_trellis_b200 needs a CUDA device; there is no CPU path")
        self.device = torch.cuda.current_device() if device is None else int(device)
        torch.cuda.set_device(self.device)
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make sure the primary context exists
        desc = N.ContextDesc()
        desc.struct_size = C.sizeof(N.ContextDesc)
        desc.abi_version = N.ABI_VERSION
        desc.device_ordinal = self.device
        self.handle = N.vp()
        N.check(self.lib.strix_context_create(C.byref(desc), C.byref(self.handle)), "strix_context_create")

    def close(self):
        if self.handle:
            N.check(self.lib.strix_context_destroy(self.handle), "strix_context_destroy")
            self.handle = N.vp()

    def device_status(self):
        bits = N.u32()
        N.check(self.lib.strix_b200_device_status(self.handle, C.byref(bits)), "strix_b200_device_status")
        return bits.value

    def set_programmatic_launch(self, enabled):
        N.check(self.lib.strix_b200_set_programmatic_launch(self.handle, int(bool(enabled))), "set_pdl")

    def prepare(self, layer, stream=None, use_blob=False):
        return Weights(self, layer, stream, use_blob)

    def moe_combine(self, rows, scores, y, alpha=1.0, beta=0.0, stream=None):
        """y[t] = alpha * sum_s (ascending, from +0) scores[t,s] * rows[t,s,:] + beta * y[t];
        rows [T, top_k, width] and scores [T, top_k] contiguous float32 CUDA tensors."""
        tokens, top_k, width = rows.shape
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_moe_combine(self.handle, rows.data_ptr(), scores.data_ptr(), tokens, top_k, width,
                                                y.data_ptr(), y.stride(0), alpha, beta, C.byref(sd)),
                "strix_b200_moe_combine")
        return y


def _bytes_view(a, dtype):
    a = np.ascontiguousarray(np.asarray(a), dtype=dtype)
    return a, a.ctypes.data, a.nbytes


class Weights:
    """Prepared weights from anything with trellis/suh/svh/bias/bits/codebook attributes
    (synthetic.Layer or container.Exl3Tensor)."""

    def __init__(self, ctx, layer, stream=None, use_blob=False):
        self.ctx, self.lib = ctx, ctx.lib
        trellis = np.asarray(layer.trellis)
        self.inputs, self.outputs = trellis.shape[0] * 16, trellis.shape[1] * 16
        bits = float(layer.bits)
        if (2 * bits) != int(2 * bits) or not (bits.is_integer() or layer.codebook == "mul1"):
            raise ValueError("rates are 1..8, and 1.5 / 2.5 / 3.5 for mul1")
        self.bits, self.codebook = (int(bits) if bits.is_integer() else bits), layer.codebook
        self.bits_x2 = int(2 * bits)
        keep = []
        t, tp, tb = _bytes_view(trellis.view(np.uint16) if trellis.dtype.itemsize == 2 else trellis, "<u2")
        su, sup, sub = _bytes_view(layer.suh, "<f2")
        sv, svp, svb = _bytes_view(layer.svh, "<f2")
        keep += [t, su, sv]
        bp, bb = None, 0
        if layer.bias is not None:
            b, bp, bb = _bytes_view(layer.bias, "<f4")
            keep.append(b)
        sd = _cur_stream(stream)
        self.handle = N.vp()
        cb = N.CODEBOOKS.index(self.codebook)
        if use_blob:
            parts = [(tp, tb, 4), (sup, sub, 2), (svp, svb, 2)] + ([(bp, bb, 4)] if bb else [])
            blob, offsets = bytearray(), []
            for ptr, nbytes, _ in parts:
                while len(blob) % 4:
                    blob.append(0)
                offsets.append(len(blob))
                blob += C.string_at(ptr, nbytes)
            buf = (C.c_char * len(blob)).from_buffer(blob)
            m = N.Metadata()
            m.struct_size = C.sizeof(N.Metadata)
            m.transport_version = 1
            m.rows, m.columns = self.outputs, self.inputs
            m.bits_x2, m.codebook, m.marker = self.bits_x2, cb, N.MARKERS[self.codebook]
            m.trellis_offset, m.trellis_bytes = offsets[0], tb
            m.suh_offset, m.suh_bytes = offsets[1], sub
            m.svh_offset, m.svh_bytes = offsets[2], svb
            if bb:
                m.bias_offset, m.bias_bytes = offsets[3], bb
            d = N.TransportDesc()
            d.struct_size = C.sizeof(N.TransportDesc)
            d.abi_version, d.format, d.transport_version = N.ABI_VERSION, 1, 1
            d.data, d.data_bytes = C.addressof(buf), len(blob)
            d.metadata, d.metadata_bytes = C.addressof(m), C.sizeof(m)
            d.rows, d.columns = self.outputs, self.inputs
            st = self.lib.strix_weights_prepare(ctx.handle, C.byref(d), C.byref(sd), C.byref(self.handle))
            N.check(st, "strix_weights_prepare")
        else:
            d = N.PartsDesc()
            d.struct_size = C.sizeof(N.PartsDesc)
            d.abi_version, d.transport_version = N.ABI_VERSION, 1
            d.bits_x2, d.rows, d.columns = self.bits_x2, self.outputs, self.inputs
            d.codebook, d.marker = cb, N.MARKERS[self.codebook]
            d.trellis, d.suh, d.svh = N.HostRegion(tp, tb), N.HostRegion(sup, sub), N.HostRegion(svp, svb)
            d.bias = N.HostRegion(bp, bb)
            st = self.lib.strix_weights_prepare_parts(ctx.handle, C.byref(d), C.byref(sd), C.byref(self.handle))
            N.check(st, "strix_weights_prepare_parts")
        del keep
        self.packed_bytes = tb

    def close(self):
        if self.handle:
            N.check(self.lib.strix_weights_destroy(self.handle), "strix_weights_destroy")
            self.handle = N.vp()

    def device_span(self):
        p, n = N.vp(), N.u64()
        N.check(self.lib.strix_weights_device_span(self.handle, C.byref(p), C.byref(n)), "device_span")
        return p.value, n.value

    # ---- descriptors -----------------------------------------------------------------
    def matmul_desc(self, x, y, alpha=1.0, beta=0.0, workspace=None):
        d = N.MatmulDesc()
        self.lib.strix_matmul_desc_init(C.byref(d))
        d.weights = self.handle
        for t, desc_name, width in ((x, "input", self.inputs), (y, "output", self.outputs)):
            shape = tuple(t.shape)
            strides = None if t.dim() == 1 else (t.stride(0), t.stride(1))
            size = t.element_size()
            nbytes = 0 if t.numel() == 0 else ((shape[0] - 1) * t.stride(0) + shape[-1]) * size if t.dim() == 2 else t.numel() * size
            dtype = {torch.float32: N.DTYPE_F32, torch.float16: N.DTYPE_F16, torch.bfloat16: N.DTYPE_BF16}[t.dtype]
            setattr(d, desc_name, N.tensor_desc(t.data_ptr() if t.numel() else 0, nbytes, shape, strides, dtype))
        d.alpha, d.beta = alpha, beta
        if workspace is not None and workspace.numel():
            d.workspace, d.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
        return d

    def workspace_bytes(self, x, y):
        d = self.matmul_desc(x, y)
        out = N.u64()
        N.check(self.lib.strix_matmul_workspace_bytes(self.ctx.handle, C.byref(d), C.byref(out)), "workspace_bytes")
        return out.value

    def _workspace(self, x, y):
        n = self.workspace_bytes(x, y)
        return torch.empty(max(n, 1), dtype=torch.uint8, device=x.device) if n else None

    def gemv(self, x, y=None, alpha=1.0, beta=0.0, workspace=None, stream=None):
        """x, y: float32, float16 or bfloat16 CUDA tensors (each on its own); y defaults to float32."""
        if y is None:
            y = torch.empty(x.shape[:-1] + (self.outputs,), dtype=torch.float32, device=x.device)
        if workspace is None:
            workspace = self._workspace(x, y)
        d = self.matmul_desc(x, y, alpha, beta, workspace)
        sd = _cur_stream(stream)
        N.check(self.lib.strix_gemv(self.ctx.handle, C.byref(d), C.byref(sd)), "strix_gemv")
        return y

    def gemm(self, x, y=None, alpha=1.0, beta=0.0, workspace=None, stream=None):
        if y is None:
            y = torch.empty((x.shape[0], self.outputs), dtype=torch.float32, device=x.device)
        if workspace is None:
            workspace = self._workspace(x, y)
        d = self.matmul_desc(x, y, alpha, beta, workspace)
        sd = _cur_stream(stream)
        N.check(self.lib.strix_gemm(self.ctx.handle, C.byref(d), C.byref(sd)), "strix_gemm")
        return y

    def plan(self, x, y, operation=N.OP_GEMV, alpha=1.0, beta=0.0, workspace=None, stream=None):
        return LinearPlan(self, x, y, operation, alpha, beta, workspace, stream)

    # ---- stage probes -----------------------------------------------------------------
    def dequantize(self, stream=None):
        q = torch.empty((self.inputs, self.outputs), dtype=torch.float16, device="cuda")
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_dequantize(self.ctx.handle, self.handle, q.data_ptr(), q.numel() * 2,
                                               C.byref(sd)), "strix_b200_dequantize")
        return q

    def input_stages(self, x, stream=None):
        rows = x.shape[0]
        scaled = torch.empty((rows, self.inputs), dtype=torch.float16, device=x.device)
        had = torch.empty((rows, self.inputs), dtype=torch.float32, device=x.device)
        core = torch.empty((rows, self.inputs), dtype=torch.float16, device=x.device)
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_input_stages(self.ctx.handle, self.handle, x.data_ptr(), rows,
                                                 scaled.data_ptr(), had.data_ptr(), core.data_ptr(),
                                                 C.byref(sd)), "strix_b200_input_stages")
        return scaled, had, core

    def output_stages(self, core, alpha=1.0, beta=0.0, y=None, stream=None):
        splits = core.shape[0] if core.dim() == 3 else 1
        rows = core.shape[-2]
        if y is None:
            y = torch.empty((rows, self.outputs), dtype=torch.float32, device=core.device)
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_output_stages(self.ctx.handle, self.handle, core.data_ptr(), splits, rows,
                                                  alpha, beta, y.data_ptr(), C.byref(sd)),
                "strix_b200_output_stages")
        return y

    def core_exact(self, core_f16, stream=None):
        rows = core_f16.shape[0]
        out = torch.empty((rows, self.outputs), dtype=torch.float32, device=core_f16.device)
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_core_exact(self.ctx.handle, self.handle, core_f16.data_ptr(), rows,
                                               out.data_ptr(), C.byref(sd)), "strix_b200_core_exact")
        return out

    def decode_rate(self, iterations=200, warps_per_sm=16, stream=None):
        """SM clocks per 16x16 tile per SM sub-partition of the decode + mma loop alone."""
        out = C.c_double()
        sd = _cur_stream(stream)
        N.check(self.lib.strix_b200_decode_rate(self.ctx.handle, self.handle, iterations, warps_per_sm, C.byref(out),
                                                C.byref(sd)), "strix_b200_decode_rate")
        return out.value

    def gemv_splits(self, rows):
        out = N.u32()
        N.check(self.lib.strix_b200_gemv_splits(self.ctx.handle, self.handle, rows, C.byref(out)), "gemv_splits")
        return out.value


class LinearPlan:
    """strix_linear_plan: validated once, submitted many times (graph-capturable)."""

    def __init__(self, weights, x, y, operation, alpha, beta, workspace, stream):
        self.weights, self.lib = weights, weights.lib
        if workspace is None:
            workspace = weights._workspace(x, y)
        self.keep = (x, y, workspace)
        d = weights.matmul_desc(x, y, alpha, beta, workspace)
        sd = _cur_stream(stream)
        self.handle = N.vp()
        N.check(self.lib.strix_linear_plan_create(weights.ctx.handle, C.byref(d), C.byref(sd), operation,
                                                  C.byref(self.handle)), "strix_linear_plan_create")

    def submit(self):
        N.check(self.lib.strix_linear_plan_submit(self.handle), "strix_linear_plan_submit")

    def close(self):
        if self.handle:
            N.check(self.lib.strix_linear_plan_destroy(self.handle), "strix_linear_plan_destroy")
            self.handle = N.vp()


class DensePlan:
    """strix_tp_dense_plan on F32 row views (unit channel stride, any row stride, rows 1..8);
    scratch is the library's."""

    def __init__(self, weights, x, y, alpha=1.0, beta=0.0, stream=None):
        self.weights, self.lib = weights, weights.lib
        d = weights.matmul_desc(x, y, alpha, beta)
        sd = _cur_stream(stream)
        self.handle = N.vp()
        self.keep = (x, y)
        N.check(self.lib.strix_tp_dense_plan_create(weights.ctx.handle, C.byref(d), C.byref(sd), C.byref(self.handle)),
                "strix_tp_dense_plan_create")

    def submit(self):
        N.check(self.lib.strix_tp_dense_plan_submit(self.handle), "strix_tp_dense_plan_submit")

    def close(self):
        if self.handle:
            N.check(self.lib.strix_tp_dense_plan_destroy(self.handle), "strix_tp_dense_plan_destroy")
            self.handle = N.vp()


class MoePlan:
    """strix_tp_moe_plan over a list of experts [(gate, up, down) Weights].  With
    `device_routed`, `route_ids` (uint32) and `route_scores` (float32) are CUDA tensors read
    at every submit and `experts[i]` is bank entry i; otherwise they are host arrays frozen at
    creation and `expert_ids[i]` names experts[i]."""

    def __init__(self, ctx, experts, x, y, route_ids, route_scores, expert_ids=None, alpha=1.0, beta=0.0,
                 device_routed=False, stream=None):
        self.ctx, self.lib = ctx, ctx.lib
        tokens = x.shape[0]
        inter = experts[0][0].outputs
        arr = (N.ExpertDesc * len(experts))()
        for i, (g, u, d) in enumerate(experts):
            arr[i].struct_size = C.sizeof(N.ExpertDesc)
            arr[i].abi_version = N.ABI_VERSION
            arr[i].expert_id = i if expert_ids is None else int(expert_ids[i])
            arr[i].gate, arr[i].up, arr[i].down = g.handle, u.handle, d.handle
        top_k = route_ids.numel() // tokens if device_routed else np.asarray(route_ids).size // tokens
        self.workspace = torch.empty(max(tokens * top_k * inter * 4, 256), dtype=torch.uint8, device=x.device)
        sd = _cur_stream(stream)
        self.handle = N.vp()

        def tensor(t):
            nbytes = ((t.shape[0] - 1) * t.stride(0) + t.shape[1]) * 4
            return N.tensor_desc(t.data_ptr(), nbytes, tuple(t.shape), (t.stride(0), t.stride(1)))

        if device_routed:
            d = N.MoeDeviceDesc()
            self.lib.strix_tp_moe_device_desc_init(C.byref(d))
            d.route_ids, d.route_ids_bytes = route_ids.data_ptr(), route_ids.numel() * 4
            d.route_scores, d.route_scores_bytes = route_scores.data_ptr(), route_scores.numel() * 4
            create = self.lib.strix_tp_moe_plan_create_device
        else:
            d = N.MoeDesc()
            self.lib.strix_tp_moe_desc_init(C.byref(d))
            ids = np.ascontiguousarray(route_ids, dtype=np.uint32)
            sc = np.ascontiguousarray(route_scores, dtype=np.float32)
            d.route_ids, d.route_ids_count = ids.ctypes.data, ids.size
            d.route_scores, d.route_scores_count = sc.ctypes.data, sc.size
            create = self.lib.strix_tp_moe_plan_create
        d.input, d.output = tensor(x), tensor(y)
        d.experts, d.expert_count = arr, len(experts)
        d.workspace, d.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        d.alpha, d.beta = alpha, beta
        self.keep = (x, y, arr, route_ids, route_scores)
        N.check(create(ctx.handle, C.byref(d), C.byref(sd), C.byref(self.handle)), "strix_tp_moe_plan_create")
        self.tokens, self.top_k, self.inter = tokens, top_k, inter

    def submit(self):
        N.check(self.lib.strix_tp_moe_plan_submit(self.handle), "strix_tp_moe_plan_submit")

    def gate_up(self):
        N.check(self.lib.strix_tp_moe_plan_gate_up(self.handle), "strix_tp_moe_plan_gate_up")

    def down(self):
        N.check(self.lib.strix_tp_moe_plan_down(self.handle), "strix_tp_moe_plan_down")

    def hidden(self):
        return self.workspace[: self.tokens * self.top_k * self.inter * 4].view(torch.float32).view(
            self.tokens, self.top_k, self.inter)

    def gate_up_rows(self):
        """The gate and up projection rows of the last gate_up(), [tokens, top_k, intermediate]."""
        from .peer import _Raw
        g, u = N.vp(), N.vp()
        N.check(self.lib.strix_b200_moe_plan_gate_up_rows(self.handle, C.byref(g), C.byref(u)),
                "strix_b200_moe_plan_gate_up_rows")
        nbytes = self.tokens * self.top_k * self.inter * 4
        return tuple(torch.as_tensor(_Raw(p.value, nbytes), device="cuda").view(torch.float32).view(
            self.tokens, self.top_k, self.inter) for p in (g, u))

    def close(self):
        if self.handle:
            N.check(self.lib.strix_tp_moe_plan_destroy(self.handle), "strix_tp_moe_plan_destroy")
            self.handle = N.vp()
