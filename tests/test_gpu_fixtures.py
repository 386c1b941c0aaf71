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


def test_moe_route_over_a_generated_directory(tmp_path):
    """A directory in the layout of the reference's rank generator (six projection files, one
    routed window), at a small size and with the CPU contract as the source of `ref`."""
    import struct
    from oracle import c_oracle
    from strix_trellis_b200 import gpu_runtime, synthetic
    from test_fixture_reader import container
    model, inter, rows, top_k, bank = 256, 128, 8, 6, 12
    x = synthetic.make_activations(rows, model, seed=9701)
    layers = {}
    for pi, (p, i, n) in enumerate((("gate", model, inter), ("up", model, inter), ("down", inter, model))):
        for k in (2, 3):
            l = synthetic.make_layer(i, n, k, 9710 + 10 * pi + k, bias=True)
            layers[(p, k)] = l
            xin = x if p != "down" else synthetic.make_activations(rows, inter, seed=9702)
            ref = c_oracle.linear(l.trellis, l.suh, l.svh, l.bias, k, 2, xin)
            base = c_oracle.linear(l.trellis, l.suh, l.svh, None, k, 2, xin)
            meta = struct.pack("<8I", i, n, k, 2, 0x83DCD12D, rows, 1, 9710 + pi)
            sections = [("meta", meta), ("trellis", l.trellis.astype("<u2").tobytes()),
                        ("suh", l.suh.astype("<f2").tobytes()), ("svh", l.svh.astype("<f2").tobytes()),
                        ("bias", l.bias.astype("<f4").tobytes()), ("x", xin.astype("<f4").tobytes()),
                        ("old", np.zeros((rows, n), "<f4").tobytes()), ("ref", ref.tobytes()),
                        ("base", base.tobytes()), ("bound", np.full((rows, n), 1e-3, "<f8").tobytes())]
            (tmp_path / f"expert-{p}-k{k}.strank").write_bytes(container(b"STRANK01", sections))
    index = np.array([[(3 * r + s) % bank for s in range(top_k)] for r in range(rows)])
    scores = np.array([[1 + (r % 3) + s for s in range(top_k)] for r in range(rows)], "<f4")
    scores[1::3, 5] = 0
    scores /= scores.sum(axis=1, keepdims=True)
    hidden = np.zeros((rows, top_k, inter), "<f4")
    each = np.zeros((rows, top_k, model), "<f4")
    out = np.zeros((rows, model), np.float32)
    for s in range(top_k):
        for r in range(rows):
            e = int(index[r, s])
            proj = {}
            for p in ("gate", "up", "down"):
                l = layers[(p, gpu_runtime._expert_bits(e, p))]
                proj[p] = (l, gpu_runtime._expert_bias(l.bias, e, p))
            g, u = (c_oracle.linear(proj[p][0].trellis, proj[p][0].suh, proj[p][0].svh, proj[p][1],
                                    proj[p][0].bits, 2, x[r:r + 1]) for p in ("gate", "up"))
            hidden[r, s] = c_oracle.swiglu(g, u)[0]
            d = proj["down"]
            each[r, s] = c_oracle.linear(d[0].trellis, d[0].suh, d[0].svh, d[1], d[0].bits, 2, hidden[r, s][None])[0]
            if scores[r, s] != 0:
                out[r] += each[r, s] * scores[r, s]
    old = synthetic.make_activations(rows, model, seed=9703)
    meta = struct.pack("<8I", model, model, 0, 2, 0x83DCD12D, rows, 0, 9700)
    window = [("meta", meta), ("routes", (17 + 3 * index).astype("<u4").tobytes()), ("scores", scores.tobytes()),
              ("hidden", hidden.tobytes()), ("each", each.tobytes()), ("ref", out.astype("<f4").tobytes()),
              ("old", old.astype("<f4").tobytes())]
    (tmp_path / "moe-overlap.strank").write_bytes(container(b"STRANK01", window))
    log = io.StringIO()
    failures = gpu_runtime.run([tmp_path], "moe", out=log)
    assert failures == 0, "\n".join(failing(log))
    assert sum(l.startswith("PASS") and " block " in l for l in log.getvalue().splitlines()) == 4
    # the six projection files as plain matmul fixtures, held to their own bound too
    log = io.StringIO()
    assert gpu_runtime.run(sorted(tmp_path.glob("expert-*.strank")), "gemv", out=log) == 0, "\n".join(failing(log))
