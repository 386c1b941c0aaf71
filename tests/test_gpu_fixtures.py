"""The reference's external STGPU001 cases driven through the runtime on the GPU: every
route of the fixture harness (stages, GEMV, GEMM, grouped) over the committed files."""
import io
from pathlib import Path

import numpy as np
import pytest

from strix_trellis_b200 import fixtures as F

pytestmark = pytest.mark.gpu
FILES = sorted((Path(__file__).parent / "golden" / "stgpu").glob("*.stgpu"))


def failing(log):
    return [l for l in log.getvalue().splitlines() if l.startswith("FAIL")]


@pytest.mark.parametrize("route", ["stages", "gemv", "gemm", "grouped"])
def test_route_over_the_reference_fixtures(route):
    from strix_trellis_b200 import gpu_runtime
    log = io.StringIO()
    failures = gpu_runtime.run(FILES, route, out=log)
    assert failures == 0, "\n".join(failing(log)[:20])
    passed = [l for l in log.getvalue().splitlines() if l.startswith("PASS")]
    assert len(passed) >= {"stages": 9, "gemv": 50, "gemm": 60, "grouped": 40}[route] * len(FILES)


def test_harness_notices_a_wrong_reference(tmp_path):
    """Negative control: the same file with one output column of `ref` and one weight of `q`
    changed must fail the routes that read them, and the command line must exit nonzero."""
    from strix_trellis_b200 import gpu_runtime
    import struct
    sections = dict(F.read_sections(FILES[0], b"STGPU001"))
    fx = F.read_stgpu(FILES[0])
    ref = fx.ref.copy()
    ref[:, 5] += 0.25
    q = fx.q.copy()
    q[17, 3] = -q[17, 3] if q[17, 3] != 0 else np.float16(1)
    sections["ref"], sections["q"] = ref.tobytes(), q.tobytes()
    data = bytearray(b"STGPU001" + struct.pack("<II", 1, len(sections)))
    for tag, payload in sections.items():
        data += tag.encode().ljust(8, b"\0") + struct.pack("<Q", len(payload)) + payload
    bad = tmp_path / "tampered.stgpu"
    bad.write_bytes(data)
    log = io.StringIO()
    assert gpu_runtime.run([bad], "gemv", out=log) > 0
    log = io.StringIO()
    assert gpu_runtime.run([bad], "stages", out=log) > 0
    assert any("Q[" in l for l in failing(log))
    assert gpu_runtime.main(["--route", "gemv", str(bad)]) == 1
    assert gpu_runtime.main(["--route", "gemv", str(FILES[0])]) == 0
