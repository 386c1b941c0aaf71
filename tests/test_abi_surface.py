"""The shared library loads without a GPU and exports every symbol the headers declare;
the ctypes mirror of every descriptor has the size the C compiler gives it."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

from strix_trellis_b200 import native as N

ROOT = Path(__file__).resolve().parents[1]
HEADERS = [ROOT / "include" / "strix_trellis.h", ROOT / "include" / "strix_trellis_b200.h"]


def declared_symbols():
    names = set()
    for h in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names.update(re.findall(r"\b(strix_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def lib():
    if not N.library_path().exists():
        from strix_trellis_b200 import build
        build.build()
    return N.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    symbols = declared_symbols()
    assert len(symbols) >= 65
    for name in symbols:
        assert hasattr(lib, name), name
        assert name in N.PROTOTYPES, f"{name} has no ctypes prototype"
    assert sorted(N.PROTOTYPES) == symbols


def test_host_only_entry_points(lib):
    assert lib.strix_get_abi_version() == 1
    assert lib.strix_status_string(0) == b"success"
    assert lib.strix_status_string(8) == b"not implemented"
    assert lib.strix_status_string(99) == b"unknown status"
    d = N.MatmulDesc()
    lib.strix_matmul_desc_init(C.byref(d))
    assert (d.struct_size, d.abi_version, d.alpha, d.beta) == (C.sizeof(N.MatmulDesc), 1, 1.0, 0.0)
    assert d.input.dtype == N.DTYPE_F32 and d.output.struct_size == C.sizeof(N.TensorDesc)
    m = N.MoeDesc()
    lib.strix_tp_moe_desc_init(C.byref(m))
    assert m.alpha == 1.0 and m.input.rank == 2
    # argument validation that needs no device
    assert lib.strix_context_create(None, None) == N.INVALID_ARGUMENT
    out = N.vp()
    bad = N.ContextDesc()
    assert lib.strix_context_create(C.byref(bad), C.byref(out)) == N.ABI_MISMATCH
    assert lib.strix_weights_destroy(None) == N.INVALID_ARGUMENT
    assert lib.strix_linear_plan_submit(None) == N.INVALID_ARGUMENT
    p, n = N.vp(1), N.u64(1)
    assert lib.strix_weights_device_span(None, C.byref(p), C.byref(n)) == N.INVALID_ARGUMENT
    assert p.value is None and n.value == 0  # outputs cleared on error


def test_ctypes_struct_sizes_match_the_c_compiler(tmp_path):
    structs = {"strix_exl3_metadata_v1": N.Metadata, "strix_exl3_transport_desc": N.TransportDesc,
               "strix_host_region": N.HostRegion, "strix_exl3_parts_desc": N.PartsDesc,
               "strix_stream": N.Stream, "strix_context_desc": N.ContextDesc, "strix_tensor_desc": N.TensorDesc,
               "strix_matmul_desc": N.MatmulDesc, "strix_grouped_moe_desc": N.GroupedMoeDesc,
               "strix_tp_expert_desc": N.ExpertDesc, "strix_tp_moe_desc": N.MoeDesc,
               "strix_tp_moe_device_desc": N.MoeDeviceDesc, "strix_tp_dense_pair_member": N.PairMember,
               "strix_tp_dense_pair_desc": N.PairDesc, "strix_tp_swiglu_desc": N.SwigluDesc,
               "strix_grouped_gemv_desc": N.GroupedGemvDesc}
    src = tmp_path / "sizes.c"
    body = "".join(f'printf("{n} %zu\\n", sizeof({n}));' for n in structs)
    src.write_text('#include <stdio.h>\n#include "strix_trellis_b200.h"\nint main(void){' + body + "return 0;}")
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    for line in out.splitlines():
        name, size = line.split()
        assert C.sizeof(structs[name]) == int(size), name
