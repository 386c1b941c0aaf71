"""ctypes front end of the C oracle (oracle/trellis_oracle.c).  TEST INFRASTRUCTURE ONLY.

Used by tests, the smoke check and the benchmark's CPU-baseline leg; the shipped
package never imports it.  `build()` compiles the shared objects with the Makefile
beside this file when they are missing or older than their sources.
"""
import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None
_REF = None


def build(force=False):
    so, src = _HERE / "libtrellis_oracle.so", _HERE / "trellis_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s", "all"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(build()))
        _LIB.so_codebook_value.restype = ctypes.c_uint16
        _LIB.so_codebook_value.argtypes = [ctypes.c_uint32, ctypes.c_int]
        _LIB.so_max_threads.restype = ctypes.c_int
    return _LIB


def reference_host_decoder():
    """The reference's own host decoder compiled into oracle/_ref (None if absent)."""
    global _REF
    path = _HERE / "_ref" / "libref_host.so"
    if _REF is None and path.exists():
        _REF = ctypes.CDLL(str(path))
        _REF.ref_host_state.restype = ctypes.c_uint16
        _REF.ref_host_state.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        _REF.ref_host_codebook.restype = ctypes.c_uint16
        _REF.ref_host_codebook.argtypes = [ctypes.c_uint16, ctypes.c_int]
    return _REF


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _u16(a):
    a = np.asarray(a)
    if a.dtype.itemsize != 2:
        raise ValueError("expected a 16-bit array")
    return np.ascontiguousarray(a).view(np.uint16)


def codebook_table(codebook):
    out = np.empty(65536, dtype=np.uint16)
    lib().so_codebook_table(ctypes.c_int(codebook), _p(out))
    return out.view(np.float16)


def unpack_states(tile, bits):
    tile = _u16(tile)
    out = np.empty(256, dtype=np.uint16)
    lib().so_unpack_states(_p(tile), ctypes.c_int(bits), _p(out))
    return out


def dequantize(trellis, bits, codebook):
    t = _u16(trellis)
    inputs, outputs = t.shape[0] * 16, t.shape[1] * 16
    q = np.empty((inputs, outputs), dtype=np.uint16)
    lib().so_dequantize(_p(t), inputs, outputs, bits, codebook, _p(q))
    return q.view(np.float16)


def input_stages(x, suh):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, np.shape(x)[-1])
    suh = _u16(suh)
    rows, inputs = x.shape
    scaled = np.empty((rows, inputs), np.uint16)
    inh = np.empty((rows, inputs), np.float32)
    a = np.empty((rows, inputs), np.uint16)
    lib().so_input_stages(_p(x), _p(suh), rows, inputs, _p(scaled), _p(inh), _p(a))
    return {"scaled_fp16": scaled.view(np.float16), "input_hadamard_fp32": inh,
            "core_input_fp16": a.view(np.float16)}


def core_dot(a16, q16):
    a, q = _u16(a16), _u16(q16)
    rows, inputs = a.shape
    outputs = q.shape[1]
    core = np.empty((rows, outputs), np.float32)
    lib().so_core_dot(_p(a), _p(q), rows, inputs, outputs, _p(core))
    return core


def output_stages(core, svh, bias=None, alpha=1.0, beta=0.0, old=None):
    core = np.ascontiguousarray(core, dtype=np.float32)
    rows, outputs = core.shape
    svh = _u16(svh)
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    old = None if old is None else np.ascontiguousarray(old, dtype=np.float32)
    had = np.empty_like(core)
    out = np.empty_like(core)
    lib().so_output_stages(_p(core), _p(svh), _p(bias), rows, outputs, ctypes.c_float(alpha),
                           ctypes.c_float(beta), _p(old), _p(had), _p(out))
    return {"output_hadamard_fp32": had, "output": out}


def linear(trellis, suh, svh, bias, bits, codebook, x, alpha=1.0, beta=0.0, old=None,
           return_core=False):
    """alpha*Linear(x)+beta*old, streamed tile band by tile band (all host threads)."""
    t = _u16(trellis)
    inputs, outputs = t.shape[0] * 16, t.shape[1] * 16
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, inputs)
    rows = x.shape[0]
    suh, svh = _u16(suh), _u16(svh)
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    old = None if old is None else np.ascontiguousarray(old, dtype=np.float32)
    out = np.empty((rows, outputs), np.float32)
    core = np.empty((rows, outputs), np.float32) if return_core else None
    lib().so_linear(_p(t), _p(suh), _p(svh), _p(bias), inputs, outputs, bits, codebook, _p(x),
                    rows, ctypes.c_float(alpha), ctypes.c_float(beta), _p(old), _p(core), _p(out))
    return (out, core) if return_core else out


def swiglu(gate, up):
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(gate)
    lib().so_swiglu(_p(gate), _p(up), ctypes.c_size_t(gate.size), _p(out))
    return out


def threads():
    return int(os.environ.get("OMP_NUM_THREADS", lib().so_max_threads()))
