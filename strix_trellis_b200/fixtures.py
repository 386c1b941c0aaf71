"""Readers of the reference's external test containers.

Both containers share one framing (reference `docs/GPU_TESTS.md:44-68`,
`tools/make_gpu_fixtures.py:52-55`, `tools/make_rank_fixtures.py:56-69`): an 8-byte ASCII
magic, uint32 version (1), uint32 section count, then per section an 8-byte NUL-padded ASCII
tag, a uint64 length and exactly that many payload bytes.  Everything is little endian.

* ``STGPU001`` — one linear layer with every stage checkpoint of the CPU contract
  (`tools/make_gpu_fixtures.py:23-59`).
* ``STRANK01`` — one per-rank dense or expert projection with a per-output roundoff bound
  (`tools/make_rank_fixtures.py:104-124`), or a routed-expert window
  (`tools/make_rank_fixtures.py:157-200`).

The readers validate what the reference's C++ reader validates (`docs/GPU_TESTS.md:47-52`):
size limit, magic, version, duplicate and unknown-length sections, dimensions, codebook
marker, required sections, payload lengths and the absence of trailing bytes.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

MAX_FILE_BYTES = 256 << 20
CODEBOOKS = ("3inst", "mcg", "mul1")
MARKERS = (0, 0xCBAC1FED, 0x83DCD12D)


class FixtureError(ValueError):
    pass


def read_sections(path, magic):
    """The sections of a container as {tag: bytes}, in file order."""
    path = Path(path)
    size = path.stat().st_size
    if size > MAX_FILE_BYTES:
        raise FixtureError(f"{path.name}: larger than {MAX_FILE_BYTES} bytes")
    data = path.read_bytes()
    if len(data) < 16 or data[:8] != magic:
        raise FixtureError(f"{path.name}: not a {magic.decode()} container")
    version, count = struct.unpack_from("<II", data, 8)
    if version != 1:
        raise FixtureError(f"{path.name}: unsupported version {version}")
    sections, at = {}, 16
    for _ in range(count):
        if at + 16 > len(data):
            raise FixtureError(f"{path.name}: truncated section header")
        raw = data[at:at + 8]
        tag = raw.rstrip(b"\0")
        if not tag or b"\0" in tag or not tag.isascii() or raw[len(tag):].strip(b"\0"):
            raise FixtureError(f"{path.name}: malformed section tag {raw!r}")
        (length,) = struct.unpack_from("<Q", data, at + 8)
        at += 16
        if length > len(data) - at:
            raise FixtureError(f"{path.name}: section {tag.decode()} runs past the end of the file")
        name = tag.decode()
        if name in sections:
            raise FixtureError(f"{path.name}: duplicate section {name}")
        sections[name] = data[at:at + length]
        at += length
    if at != len(data):
        raise FixtureError(f"{path.name}: {len(data) - at} trailing bytes")
    return sections


def _array(sections, name, dtype, shape, path):
    payload = sections[name]
    want = int(np.prod(shape)) * np.dtype(dtype).itemsize
    if len(payload) != want:
        raise FixtureError(f"{path}: section {name} holds {len(payload)} bytes, expected {want}")
    return np.frombuffer(payload, dtype=dtype).reshape(shape)


@dataclass
class Meta:
    inputs: int
    outputs: int
    bits: int
    codebook: str
    marker: int
    rows: int
    has_bias: bool
    seed: int


def _meta(sections, path, allow_zero_bits=False):
    if "meta" not in sections or len(sections["meta"]) != 32:
        raise FixtureError(f"{path}: meta section missing or not 8 uint32")
    i, n, bits, cb, marker, rows, has_bias, seed = struct.unpack("<8I", sections["meta"])
    if cb >= len(CODEBOOKS) or marker != MARKERS[cb]:
        raise FixtureError(f"{path}: codebook {cb} with marker {marker:#x}")
    if i == 0 or n == 0 or i % 128 or n % 128:
        raise FixtureError(f"{path}: dimensions {i}x{n} are not positive multiples of 128")
    if not (1 <= bits <= 8 or (allow_zero_bits and bits == 0)):
        raise FixtureError(f"{path}: {bits} bits per weight")
    if has_bias > 1:
        raise FixtureError(f"{path}: bias flag {has_bias}")
    return Meta(i, n, bits, CODEBOOKS[cb], marker, rows, bool(has_bias), seed)


def _require(sections, names, path):
    missing = [n for n in names if n not in sections]
    if missing:
        raise FixtureError(f"{path}: missing sections {missing}")


@dataclass
class GpuFixture:
    """One STGPU001 case.  Attribute names of the layer part (trellis, suh, svh, bias, bits,
    codebook) are the ones `runtime.Context.prepare` reads."""
    name: str
    meta: Meta
    trellis: np.ndarray  # u16 [I/16, N/16, 16*bits]
    suh: np.ndarray      # f16 [I]
    svh: np.ndarray      # f16 [N]
    bias: np.ndarray | None  # f32 [N]
    x: np.ndarray        # f32 [rows, I]
    old: np.ndarray      # f32 [rows, N]
    scaled: np.ndarray   # f16 [rows, I]   RN16(x * suh)
    inh: np.ndarray      # f32 [rows, I]   H128 of scaled
    a: np.ndarray        # f16 [rows, I]   core input
    q: np.ndarray        # f16 [I, N]      decoded weight, logical order
    core: np.ndarray     # f32 [rows, N]   ordered CPU product of a and q
    ref: np.ndarray      # f32 [rows, N]   Linear(x) with bias

    @property
    def bits(self):
        return self.meta.bits

    @property
    def codebook(self):
        return self.meta.codebook


def read_stgpu(path):
    path = Path(path)
    s = read_sections(path, b"STGPU001")
    _require(s, ("meta", "trellis", "suh", "svh", "bias", "x", "old", "scaled", "inh", "a", "q", "core", "ref"),
             path.name)
    m = _meta(s, path.name)
    i, n, r = m.inputs, m.outputs, m.rows
    if m.has_bias != (len(s["bias"]) != 0):
        raise FixtureError(f"{path.name}: bias flag disagrees with the bias section")
    arr = lambda name, dtype, shape: _array(s, name, dtype, shape, path.name)
    return GpuFixture(
        path.stem, m, arr("trellis", "<u2", (i // 16, n // 16, 16 * m.bits)), arr("suh", "<f2", (i,)),
        arr("svh", "<f2", (n,)), arr("bias", "<f4", (n,)) if m.has_bias else None, arr("x", "<f4", (r, i)),
        arr("old", "<f4", (r, n)), arr("scaled", "<f2", (r, i)), arr("inh", "<f4", (r, i)), arr("a", "<f2", (r, i)),
        arr("q", "<f2", (i, n)), arr("core", "<f4", (r, n)), arr("ref", "<f4", (r, n)))


@dataclass
class RankFixture:
    """One STRANK01 projection: `ref` = Linear(x) with this file's bias, `base` the same
    without the bias, `bound` the per-output roundoff allowance (binary64)."""
    name: str
    meta: Meta
    trellis: np.ndarray
    suh: np.ndarray
    svh: np.ndarray
    bias: np.ndarray
    x: np.ndarray
    old: np.ndarray
    ref: np.ndarray
    base: np.ndarray
    bound: np.ndarray

    @property
    def bits(self):
        return self.meta.bits

    @property
    def codebook(self):
        return self.meta.codebook


@dataclass
class RouteWindowFixture:
    """One STRANK01 routed-expert window: expert ids and scores per (row, slot), the
    SwiGLU values and down outputs of every slot, and the combined block output."""
    name: str
    meta: Meta
    routes: np.ndarray  # u32 [rows, top_k]
    scores: np.ndarray  # f32 [rows, top_k]
    hidden: np.ndarray  # f32 [rows, top_k, intermediate]
    each: np.ndarray    # f32 [rows, top_k, model]
    ref: np.ndarray     # f32 [rows, model]
    old: np.ndarray     # f32 [rows, model]


def read_strank(path):
    path = Path(path)
    s = read_sections(path, b"STRANK01")
    if "routes" in s:
        _require(s, ("meta", "routes", "scores", "hidden", "each", "ref", "old"), path.name)
        m = _meta(s, path.name, allow_zero_bits=True)
        rows, model = m.rows, m.outputs
        if rows == 0 or len(s["routes"]) % (4 * rows):
            raise FixtureError(f"{path.name}: routes section does not divide into {rows} rows")
        top_k = len(s["routes"]) // (4 * rows)
        if top_k == 0 or len(s["hidden"]) % (4 * rows * top_k):
            raise FixtureError(f"{path.name}: hidden section does not divide into {rows}x{top_k} slots")
        inter = len(s["hidden"]) // (4 * rows * top_k)
        arr = lambda name, dtype, shape: _array(s, name, dtype, shape, path.name)
        return RouteWindowFixture(path.stem, m, arr("routes", "<u4", (rows, top_k)),
                                  arr("scores", "<f4", (rows, top_k)), arr("hidden", "<f4", (rows, top_k, inter)),
                                  arr("each", "<f4", (rows, top_k, model)), arr("ref", "<f4", (rows, model)),
                                  arr("old", "<f4", (rows, model)))
    _require(s, ("meta", "trellis", "suh", "svh", "bias", "x", "old", "ref", "base", "bound"), path.name)
    m = _meta(s, path.name)
    i, n, r = m.inputs, m.outputs, m.rows
    arr = lambda name, dtype, shape: _array(s, name, dtype, shape, path.name)
    return RankFixture(path.stem, m, arr("trellis", "<u2", (i // 16, n // 16, 16 * m.bits)), arr("suh", "<f2", (i,)),
                       arr("svh", "<f2", (n,)), arr("bias", "<f4", (n,)), arr("x", "<f4", (r, i)),
                       arr("old", "<f4", (r, n)), arr("ref", "<f4", (r, n)), arr("base", "<f4", (r, n)),
                       arr("bound", "<f8", (r, n)))


def read_fixture(path):
    """Dispatch on the magic."""
    with open(path, "rb") as f:
        magic = f.read(8)
    if magic == b"STGPU001":
        return read_stgpu(path)
    if magic == b"STRANK01":
        return read_strank(path)
    raise FixtureError(f"{Path(path).name}: unknown container magic {magic!r}")
