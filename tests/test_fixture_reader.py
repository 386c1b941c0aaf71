"""STGPU001 / STRANK01 containers: the committed files were written by the reference's own
generator from its CPU contract, so every stage section pins the oracle bit for bit; the
reader must also refuse what the reference's reader refuses."""
import hashlib
import json
import struct
from pathlib import Path

import numpy as np
import pytest

from oracle import c_oracle, trellis_ref
from strix_trellis_b200 import fixtures as F

STGPU = Path(__file__).parent / "golden" / "stgpu"
FILES = sorted(STGPU.glob("*.stgpu"))


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype.itemsize == b.dtype.itemsize and a.tobytes() == b.tobytes()


def test_manifest_matches_the_files():
    manifest = json.loads((STGPU / "manifest.json").read_text())
    assert manifest["format"] == "STGPU001" and len(manifest["fixtures"]) == len(FILES) == 6
    for r in manifest["fixtures"]:
        data = (STGPU / r["file"]).read_bytes()
        assert len(data) == r["bytes"] and hashlib.sha256(data).hexdigest() == r["sha256"]
        fx = F.read_stgpu(STGPU / r["file"])
        assert (fx.meta.inputs, fx.meta.outputs, fx.bits, fx.codebook, fx.meta.rows, fx.meta.seed) == \
            (r["input"], r["output"], r["bits"], r["codebook"], r["rows"], r["seed"])
        assert (fx.bias is not None) == r["bias"] == bool(fx.bits % 2)


@pytest.mark.parametrize("path", FILES, ids=lambda p: p.stem)
def test_oracles_reproduce_every_stage_of_the_reference(path):
    fx = F.read_stgpu(path)
    cb = F.CODEBOOKS.index(fx.codebook)
    # C restatement
    assert bits_equal(c_oracle.dequantize(fx.trellis, fx.bits, cb), fx.q)
    st = c_oracle.input_stages(fx.x, fx.suh)
    assert bits_equal(st["scaled_fp16"], fx.scaled)
    assert bits_equal(st["input_hadamard_fp32"], fx.inh)
    assert bits_equal(st["core_input_fp16"], fx.a)
    assert bits_equal(c_oracle.core_dot(fx.a, fx.q), fx.core)
    assert bits_equal(c_oracle.output_stages(fx.core, fx.svh, fx.bias)["output"], fx.ref)
    out, core = c_oracle.linear(fx.trellis, fx.suh, fx.svh, fx.bias, fx.bits, cb, fx.x, return_core=True)
    assert bits_equal(core, fx.core) and bits_equal(out, fx.ref)
    # NumPy restatement
    ref = trellis_ref.linear_stages(fx.x, fx.trellis, fx.suh, fx.svh, fx.bits, fx.codebook, fx.bias)
    for name, want in (("rotated_fp16", fx.q), ("scaled_fp16", fx.scaled), ("input_hadamard_fp32", fx.inh),
                       ("core_input_fp16", fx.a), ("core_fp32", fx.core), ("output_fp32", fx.ref)):
        assert bits_equal(ref[name], want), name


def test_first_row_is_the_impulse_probe():
    fx = F.read_stgpu(FILES[0])
    cols = [0, 1, 31, 32, 63, 64, 127, fx.meta.inputs - 1]
    assert np.count_nonzero(fx.x[0]) == len(cols) and np.all(fx.x[0, cols] != 0)


def container(magic, sections, version=1, count=None, tail=b""):
    out = bytearray(magic + struct.pack("<II", version, len(sections) if count is None else count))
    for tag, payload in sections:
        out += tag.encode().ljust(8, b"\0") + struct.pack("<Q", len(payload)) + payload
    return bytes(out + tail)


def sections_of(path):
    return list(F.read_sections(path, b"STGPU001").items())


def test_reader_refuses_malformed_containers(tmp_path):
    good = sections_of(FILES[0])
    p = tmp_path / "case.stgpu"

    def refuse(data, match):
        p.write_bytes(data)
        with pytest.raises(F.FixtureError, match=match):
            F.read_stgpu(p)

    p.write_bytes(container(b"STGPU001", good))
    assert F.read_stgpu(p).meta.rows == 32  # the rebuilt container itself is fine
    refuse(container(b"STGPU002", good), "not a STGPU001")
    refuse(container(b"STGPU001", good, version=2), "version")
    refuse(container(b"STGPU001", good, tail=b"\0"), "trailing")
    refuse(container(b"STGPU001", good)[:-5], "past the end")
    refuse(container(b"STGPU001", good, count=len(good) + 1), "truncated")
    refuse(container(b"STGPU001", good + [good[3]]), "duplicate")
    refuse(container(b"STGPU001", [s for s in good if s[0] != "core"]), "missing")
    refuse(container(b"STGPU001", [(t, v[:-2] if t == "x" else v) for t, v in good]), "section x holds")
    meta = list(struct.unpack("<8I", dict(good)["meta"]))

    def with_meta(**kw):
        m = list(meta)
        for k, v in kw.items():
            m[("inputs", "outputs", "bits", "codebook", "marker", "rows", "bias", "seed").index(k)] = v
        return container(b"STGPU001", [(t, struct.pack("<8I", *m) if t == "meta" else v) for t, v in good])

    refuse(with_meta(marker=0x1234), "marker")
    refuse(with_meta(codebook=3), "codebook")
    refuse(with_meta(inputs=meta[0] + 16), "multiples of 128")
    refuse(with_meta(bits=9), "bits")
    refuse(with_meta(bias=1 - meta[6]), "bias flag")
    refuse(with_meta(rows=meta[5] + 1), "holds")
    refuse(container(b"STGPU001", [("bad\0tag", b"")] + good), "malformed")
    with pytest.raises(F.FixtureError, match="unknown container"):
        p.write_bytes(b"SOMETHING" + bytes(16))
        F.read_fixture(p)


def test_rank_containers(tmp_path):
    """STRANK01 framing and section set (written here in the generator's layout: the
    generator's own files are tens of megabytes)."""
    fx = F.read_stgpu(FILES[-1])  # mul1, odd rate: has a bias
    assert fx.codebook == "mul1" and fx.bias is not None
    rows = 8
    ref = c_oracle.linear(fx.trellis, fx.suh, fx.svh, fx.bias, fx.bits, 2, fx.x[:rows])
    base = c_oracle.linear(fx.trellis, fx.suh, fx.svh, None, fx.bits, 2, fx.x[:rows])
    bound = np.full(ref.shape, 1e-3, "<f8")
    meta = struct.pack("<8I", fx.meta.inputs, fx.meta.outputs, fx.bits, 2, 0x83DCD12D, rows, 1, 77)
    dense = [("meta", meta), ("trellis", fx.trellis.tobytes()), ("suh", fx.suh.tobytes()), ("svh", fx.svh.tobytes()),
             ("bias", fx.bias.tobytes()), ("x", fx.x[:rows].tobytes()), ("old", fx.old[:rows].tobytes()),
             ("ref", ref.tobytes()), ("base", base.tobytes()), ("bound", bound.tobytes())]
    p = tmp_path / "dense-case-k5.strank"
    p.write_bytes(container(b"STRANK01", dense))
    got = F.read_fixture(p)
    assert isinstance(got, F.RankFixture) and got.meta.seed == 77 and got.bits == fx.bits
    assert bits_equal(got.ref, ref) and bits_equal(got.base, base) and got.bound.dtype == np.float64
    assert bits_equal(got.trellis, fx.trellis)
    p.write_bytes(container(b"STRANK01", dense[:-1]))
    with pytest.raises(F.FixtureError, match="missing"):
        F.read_strank(p)
    # routed-expert window: bits field is 0, widths come from the section lengths
    top_k, inter, model = 6, 128, 256
    rng = np.random.default_rng(5)
    routes = (17 + 3 * rng.integers(0, 12, (rows, top_k))).astype("<u4")
    scores = rng.random((rows, top_k)).astype("<f4")
    hidden = rng.standard_normal((rows, top_k, inter)).astype("<f4")
    each = rng.standard_normal((rows, top_k, model)).astype("<f4")
    out = rng.standard_normal((rows, model)).astype("<f4")
    meta = struct.pack("<8I", model, model, 0, 2, 0x83DCD12D, rows, 0, 9)
    window = [("meta", meta), ("routes", routes.tobytes()), ("scores", scores.tobytes()),
              ("hidden", hidden.tobytes()), ("each", each.tobytes()), ("ref", out.tobytes()), ("old", out.tobytes())]
    p.write_bytes(container(b"STRANK01", window))
    got = F.read_fixture(p)
    assert isinstance(got, F.RouteWindowFixture)
    assert got.routes.shape == (rows, top_k) and got.hidden.shape == (rows, top_k, inter)
    assert bits_equal(got.each, each) and bits_equal(got.scores, scores)


def test_harness_expectation_and_criterion():
    """Host side of the fixture harness: alpha/beta applied with separate roundings, a zero
    beta of either sign never reads the old output, and the two-part criterion."""
    import io
    from strix_trellis_b200 import gpu_runtime as G
    ref = np.array([[1.0, -2.5, 3.0e-3]], np.float32)
    old = np.array([[np.nan, np.inf, 7.0]], np.float32)
    for beta in (0.0, -0.0):
        assert bits_equal(G.expected(ref, old, -0.75, beta), (np.float32(-0.75) * ref).astype(np.float32))
    old = np.array([[0.1, 0.2, 0.3]], np.float32)
    want = trellis_ref.apply_alpha_beta(ref, -0.75, 0.25, old)
    assert bits_equal(G.expected(ref, old, -0.75, 0.25), want)
    rep = G.Report(io.StringIO())
    rep.tolerance("exact", ref, ref)
    rep.tolerance("inside", ref + np.float32(2e-6), ref)
    assert rep.failures == 0
    rep.tolerance("maxabs", ref + np.array([[0, 0, 2e-3]], np.float32), ref)      # 2e-3 > 5e-4*max(1, 2.5)
    rep.tolerance("nrmse", ref + np.float32(2e-4), ref)                            # inside maxabs, NRMSE 8.9e-5
    rep.tolerance("nan", np.array([[1.0, np.nan, 0.0]], np.float32), ref)
    rep.tolerance("bound", ref + np.float32(2e-6), ref, bound=np.full(ref.shape, 1e-6))
    rep.identical("bytes", np.float32([0.0]), np.float32([-0.0]))                  # signed zeros count
    assert rep.failures == 5 and rep.checks == 7
    assert [G._expert_bits(i, p) for i in range(3) for p in ("gate", "up", "down")] == [2, 3, 3, 3, 2, 2, 2, 2, 3]
    assert G._expert_index(17 + 3 * 11) == 11
    assert G._expert_bias(np.zeros(2, np.float32), 1, "up")[0] == np.float32(-21 * 0.5 / 512)
