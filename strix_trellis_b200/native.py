"""ctypes binding of libstrix_trellis.so: the descriptor structs of
include/strix_trellis.h and typed prototypes for every exported entry point.

The reference ships no Python binding for its native library ("Python HIP bindings:
None", reference README.md:181); this module is what a Python caller of the C ABI
uses.  It fails loudly when the library is missing -- there is no fallback.
"""
import ctypes as C
from pathlib import Path

ABI_VERSION = 1
ALIGN = 256
MARKERS = {"3inst": 0, "mcg": 0xCBAC1FED, "mul1": 0x83DCD12D}
CODEBOOKS = ("3inst", "mcg", "mul1")
DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 1, 2, 3
OP_GEMV, OP_GEMM = 0, 1

STATUS_NAMES = ["SUCCESS", "INVALID_ARGUMENT", "ABI_MISMATCH", "UNSUPPORTED_FORMAT",
                "UNSUPPORTED_DEVICE", "INSUFFICIENT_BUFFER", "OUT_OF_MEMORY", "BACKEND",
                "NOT_IMPLEMENTED"]
(SUCCESS, INVALID_ARGUMENT, ABI_MISMATCH, UNSUPPORTED_FORMAT, UNSUPPORTED_DEVICE,
 INSUFFICIENT_BUFFER, OUT_OF_MEMORY, BACKEND, NOT_IMPLEMENTED) = range(9)


class StrixError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{where}: STRIX_{'ERROR_' if status else ''}{name}")


u32, u64, i32, f32, vp = C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_void_p


class Metadata(C.Structure):
    _fields_ = [("struct_size", u32), ("transport_version", u32), ("rows", u64), ("columns", u64),
                ("bits_x2", u32), ("codebook", u32), ("marker", u32), ("flags", u32),
                ("trellis_offset", u64), ("trellis_bytes", u64), ("suh_offset", u64), ("suh_bytes", u64),
                ("svh_offset", u64), ("svh_bytes", u64), ("bias_offset", u64), ("bias_bytes", u64),
                ("reserved", u64 * 4)]


class TransportDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("format", u32), ("transport_version", u32),
                ("data", vp), ("data_bytes", u64), ("metadata", vp), ("metadata_bytes", u64),
                ("rows", u64), ("columns", u64), ("reserved", u64 * 4)]


class HostRegion(C.Structure):
    _fields_ = [("data", vp), ("bytes", u64)]


class PartsDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("transport_version", u32), ("bits_x2", u32),
                ("rows", u64), ("columns", u64), ("codebook", u32), ("marker", u32),
                ("trellis", HostRegion), ("suh", HostRegion), ("svh", HostRegion), ("bias", HostRegion),
                ("reserved", u64 * 4)]


class Stream(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("hip_stream", vp), ("reserved", u64 * 2)]


class ContextDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("device_ordinal", i32), ("flags", u32),
                ("reserved", u64 * 4)]


class TensorDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("data", vp), ("buffer_bytes", u64),
                ("dtype", u32), ("rank", u32), ("shape", u64 * 2), ("strides", u64 * 2),
                ("reserved", u64 * 4)]


class MatmulDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("weights", vp), ("input", TensorDesc),
                ("output", TensorDesc), ("alpha", f32), ("beta", f32), ("workspace", vp),
                ("workspace_bytes", u64), ("reserved", u64 * 4)]


class GroupedMoeDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("groups", C.POINTER(MatmulDesc)),
                ("group_count", u64), ("workspace", vp), ("workspace_bytes", u64), ("reserved", u64 * 4)]


class ExpertDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("expert_id", u32), ("flags", u32),
                ("gate", vp), ("up", vp), ("down", vp), ("reserved", u64 * 2)]


class MoeDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("input", TensorDesc), ("output", TensorDesc),
                ("experts", C.POINTER(ExpertDesc)), ("expert_count", u64),
                ("route_ids", vp), ("route_ids_count", u64), ("route_scores", vp), ("route_scores_count", u64),
                ("workspace", vp), ("workspace_bytes", u64), ("alpha", f32), ("beta", f32),
                ("reserved", u64 * 4)]


class MoeDeviceDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("input", TensorDesc), ("output", TensorDesc),
                ("experts", C.POINTER(ExpertDesc)), ("expert_count", u64),
                ("route_ids", vp), ("route_ids_bytes", u64), ("route_scores", vp), ("route_scores_bytes", u64),
                ("workspace", vp), ("workspace_bytes", u64), ("alpha", f32), ("beta", f32),
                ("reserved", u64 * 4)]


class PairMember(C.Structure):
    _fields_ = [("weights", vp), ("output", TensorDesc), ("alpha", f32), ("beta", f32)]


class PairDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("input", TensorDesc), ("member", PairMember * 2),
                ("workspace", vp), ("workspace_bytes", u64), ("rows_per_block", u32), ("strategy", u32),
                ("reserved", u64 * 4)]


class SwigluDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("input", TensorDesc), ("gate", vp), ("up", vp),
                ("hidden_output", TensorDesc), ("workspace", vp), ("workspace_bytes", u64),
                ("rows_per_block", u32), ("strategy", u32), ("diagnostic_gate", vp), ("diagnostic_up", vp),
                ("diagnostic_bytes", u64), ("reserved", u64 * 4)]


class GroupedGemvDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("weights", C.POINTER(vp)), ("group_count", u64),
                ("rows", u32), ("flags", u32), ("input", vp), ("input_row_stride", u64),
                ("input_group_stride", u64), ("input_buffer_bytes", u64), ("output", vp),
                ("output_row_stride", u64), ("output_group_stride", u64), ("output_buffer_bytes", u64),
                ("workspace", vp), ("workspace_bytes", u64), ("reserved", u64 * 4)]


P = C.POINTER
# name -> (restype, argtypes).  Every symbol declared in include/*.h is listed here;
# tests check that the library exports each of them.
PEER_RANKS, PEER_HANDLE_BYTES, PEER_CONTROL_BYTES = 8, 64, 2304
PEER_GATHER_TAGGED = 1


class PeerMatrix(C.Structure):
    _fields_ = [("block", vp * PEER_RANKS), ("result", vp * PEER_RANKS), ("width", u32 * PEER_RANKS),
                ("col_at", u32 * PEER_RANKS), ("total_cols", u64), ("region", u64)]


class PeerGatherDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("matrices", u32), ("flags", u32),
                ("rows", u32 * PEER_RANKS), ("row_at", u32 * PEER_RANKS), ("matrix", PeerMatrix * 3),
                ("reserved", u64 * 2)]


class PeerReturnDesc(C.Structure):
    _fields_ = [("struct_size", u32), ("abi_version", u32), ("each", vp * PEER_RANKS), ("ids", vp * PEER_RANKS),
                ("row_valid", vp * PEER_RANKS), ("first_expert", u32 * PEER_RANKS), ("experts", u32 * PEER_RANKS),
                ("tokens", u32), ("tokens_per_rank", u32), ("top_k", u32), ("flags", u32), ("width", u64),
                ("region", u64), ("reserved", u64 * 2)]


PROTOTYPES = {
    "strix_get_abi_version": (u32, []),
    "strix_status_string": (C.c_char_p, [C.c_int]),
    "strix_matmul_desc_init": (None, [P(MatmulDesc)]),
    "strix_context_create": (C.c_int, [P(ContextDesc), P(vp)]),
    "strix_context_destroy": (C.c_int, [vp]),
    "strix_weights_prepare": (C.c_int, [vp, P(TransportDesc), P(Stream), P(vp)]),
    "strix_weights_prepare_parts": (C.c_int, [vp, P(PartsDesc), P(Stream), P(vp)]),
    "strix_weights_destroy": (C.c_int, [vp]),
    "strix_weights_device_span": (C.c_int, [vp, P(vp), P(u64)]),
    "strix_matmul_workspace_bytes": (C.c_int, [vp, P(MatmulDesc), P(u64)]),
    "strix_gemv": (C.c_int, [vp, P(MatmulDesc), P(Stream)]),
    "strix_gemm": (C.c_int, [vp, P(MatmulDesc), P(Stream)]),
    "strix_linear_plan_create": (C.c_int, [vp, P(MatmulDesc), P(Stream), u32, P(vp)]),
    "strix_linear_plan_submit": (C.c_int, [vp]),
    "strix_linear_plan_destroy": (C.c_int, [vp]),
    "strix_grouped_moe_workspace_bytes": (C.c_int, [vp, P(GroupedMoeDesc), P(u64)]),
    "strix_grouped_moe": (C.c_int, [vp, P(GroupedMoeDesc), P(Stream)]),
    "strix_tp_dense_plan_create": (C.c_int, [vp, P(MatmulDesc), P(Stream), P(vp)]),
    "strix_tp_dense_plan_create_tiled": (C.c_int, [vp, P(MatmulDesc), P(Stream), u32, P(vp)]),
    "strix_tp_dense_workspace_bytes": (C.c_int, [vp, P(MatmulDesc), u32, P(u64)]),
    "strix_tp_dense_plan_create_splitk": (C.c_int, [vp, P(MatmulDesc), P(Stream), u32, u32, P(vp)]),
    "strix_tp_dense_pair_desc_init": (None, [P(PairDesc)]),
    "strix_tp_swiglu_desc_init": (None, [P(SwigluDesc)]),
    "strix_tp_dense_pair_workspace_bytes": (C.c_int, [vp, P(PairDesc), P(u64)]),
    "strix_tp_dense_pair_plan_create": (C.c_int, [vp, P(PairDesc), P(Stream), P(vp)]),
    "strix_tp_dense_pair_plan_submit": (C.c_int, [vp]),
    "strix_tp_dense_pair_plan_destroy": (C.c_int, [vp]),
    "strix_tp_swiglu_workspace_bytes": (C.c_int, [vp, P(SwigluDesc), P(u64)]),
    "strix_tp_swiglu_plan_create": (C.c_int, [vp, P(SwigluDesc), P(Stream), P(vp)]),
    "strix_tp_swiglu_plan_submit": (C.c_int, [vp]),
    "strix_tp_swiglu_plan_destroy": (C.c_int, [vp]),
    "strix_tp_dense_r1_workspace_bytes": (C.c_int, [vp, P(MatmulDesc), u32, u32, P(u64)]),
    "strix_tp_dense_plan_create_r1": (C.c_int, [vp, P(MatmulDesc), P(Stream), u32, u32, P(vp)]),
    "strix_tp_dense_plan_submit": (C.c_int, [vp]),
    "strix_tp_dense_plan_destroy": (C.c_int, [vp]),
    "strix_tp_dense_pair_r1_workspace_bytes": (C.c_int, [vp, P(PairDesc), u32, P(u64)]),
    "strix_tp_dense_pair_plan_create_r1": (C.c_int, [vp, P(PairDesc), P(Stream), u32, P(vp)]),
    "strix_grouped_gemv_workspace_bytes": (C.c_int, [vp, P(GroupedGemvDesc), P(u64)]),
    "strix_grouped_gemv_plan_create": (C.c_int, [vp, P(GroupedGemvDesc), P(Stream), P(vp)]),
    "strix_grouped_gemv_plan_submit": (C.c_int, [vp]),
    "strix_grouped_gemv_plan_destroy": (C.c_int, [vp]),
    "strix_tp_moe_desc_init": (None, [P(MoeDesc)]),
    "strix_tp_moe_device_desc_init": (None, [P(MoeDeviceDesc)]),
    "strix_tp_moe_workspace_bytes": (C.c_int, [vp, P(MoeDesc), P(u64)]),
    "strix_tp_moe_plan_create": (C.c_int, [vp, P(MoeDesc), P(Stream), P(vp)]),
    "strix_tp_moe_plan_create_device": (C.c_int, [vp, P(MoeDeviceDesc), P(Stream), P(vp)]),
    "strix_tp_moe_split_workspace_bytes": (C.c_int, [vp, P(MoeDesc), P(u64)]),
    "strix_tp_moe_plan_create_split": (C.c_int, [vp, P(MoeDesc), P(Stream), P(vp)]),
    "strix_tp_moe_plan_create_device_split": (C.c_int, [vp, P(MoeDeviceDesc), P(Stream), P(vp)]),
    "strix_tp_moe_plan_create_a8r": (C.c_int, [vp, P(MoeDesc), P(Stream), P(vp)]),
    "strix_tp_moe_plan_create_device_a8r": (C.c_int, [vp, P(MoeDeviceDesc), P(Stream), P(vp)]),
    "strix_tp_moe_plan_down_core": (C.c_int, [vp]),
    "strix_tp_moe_plan_down_finish": (C.c_int, [vp]),
    "strix_tp_moe_plan_down_reference_core": (C.c_int, [vp]),
    "strix_tp_moe_plan_submit": (C.c_int, [vp]),
    "strix_tp_moe_plan_gate_up": (C.c_int, [vp]),
    "strix_tp_moe_plan_down": (C.c_int, [vp]),
    "strix_tp_moe_plan_destroy": (C.c_int, [vp]),
    # strix_trellis_b200.h
    "strix_b200_dequantize": (C.c_int, [vp, vp, vp, u64, P(Stream)]),
    "strix_b200_input_stages": (C.c_int, [vp, vp, vp, u32, vp, vp, vp, P(Stream)]),
    "strix_b200_output_stages": (C.c_int, [vp, vp, vp, u32, u32, f32, f32, vp, P(Stream)]),
    "strix_b200_core_exact": (C.c_int, [vp, vp, vp, u32, vp, P(Stream)]),
    "strix_b200_decode_rate": (C.c_int, [vp, vp, u32, u32, P(C.c_double), P(Stream)]),
    "strix_b200_gemv_splits": (C.c_int, [vp, vp, u32, P(u32)]),
    "strix_b200_gemv_partition": (C.c_int, [u64, u64, u32, u32, u64, P(u64)]),
    "strix_b200_moe_combine": (C.c_int, [vp, vp, vp, u32, u32, u32, vp, u64, f32, f32, P(Stream)]),
    "strix_b200_moe_combine_rows": (C.c_int, [vp, vp, vp, vp, u32, u32, u32, vp, u64, f32, f32, P(Stream)]),
    "strix_b200_moe_plan_set_window": (C.c_int, [vp, u32, u32]),
    "strix_b200_moe_plan_projections": (C.c_int, [vp]),
    "strix_b200_moe_plan_rows": (C.c_int, [vp, P(vp), P(vp)]),
    "strix_b200_moe_plan_gate_up_rows": (C.c_int, [vp, P(vp), P(vp)]),
    "strix_b200_peer_group_set_wait_polls": (C.c_int, [vp, C.c_uint32]),
    "strix_b200_peer_arena_create": (C.c_int, [vp, u64, P(vp), C.c_char_p]),
    "strix_b200_peer_arena_destroy": (C.c_int, [vp, vp]),
    "strix_b200_peer_group_create": (C.c_int, [vp, P(vp), u32, u32, u64, C.c_char_p, u32, P(vp)]),
    "strix_b200_peer_group_destroy": (C.c_int, [vp]),
    "strix_b200_peer_sum": (C.c_int, [vp, P(vp), u64, u64, P(Stream)]),
    "strix_b200_peer_gather": (C.c_int, [vp, P(PeerGatherDesc), P(Stream)]),
    "strix_b200_peer_return_routes": (C.c_int, [vp, P(PeerReturnDesc), P(Stream)]),
    "strix_b200_device_status": (C.c_int, [vp, P(u32)]),
    "strix_b200_set_programmatic_launch": (C.c_int, [vp, u32]),
    "strix_b200_gemv_noalloc": (C.c_int, [vp, P(MatmulDesc), P(Stream)]),
}

_LIB = None


def library_path():
    return Path(__file__).resolve().parent / "libstrix_trellis.so"


def load(path=None):
    """Load the shared library and attach prototypes.  Raises if it is absent."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    p = Path(path) if path else library_path()
    if not p.exists():
        raise FileNotFoundError(
            f"{p} is missing: build it with `python -m strix_trellis_b200.build` (needs nvcc). "
            "There is no CPU fallback.")
    lib = C.CDLL(str(p))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _LIB = lib
    return lib


def check(status, where):
    if status != SUCCESS:
        raise StrixError(status, where)


def stream_desc(cuda_stream=0):
    s = Stream()
    s.struct_size = C.sizeof(Stream)
    s.abi_version = ABI_VERSION
    s.hip_stream = cuda_stream or None
    return s


def tensor_desc(ptr, nbytes, shape, strides=None, dtype=None):
    t = TensorDesc()
    t.struct_size = C.sizeof(TensorDesc)
    t.abi_version = ABI_VERSION
    t.data = ptr or None
    t.buffer_bytes = nbytes
    t.dtype = DTYPE_F32 if dtype is None else dtype
    t.rank = len(shape)
    if len(shape) == 1:
        t.shape[0], t.shape[1] = shape[0], 0
        t.strides[0], t.strides[1] = 1, 0
    else:
        t.shape[0], t.shape[1] = shape
        t.strides[0], t.strides[1] = strides if strides else (shape[1], 1)
    return t
