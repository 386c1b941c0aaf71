"""EXL3 tensor groups read from local safetensors files through memory maps, and their
export as the four transport regions that strix_weights_prepare[_parts] consumes.

The public names and their behaviour follow the loader the reference documents in
docs/LOADER.md and docs/FORMAT.md (python/strix_trellis/container.py: SafetensorsFile,
Exl3Tensor, load_exl3): what is accepted, what raises ValueError, which arrays are borrowed
and which are packed.  The implementation here is organised differently: one header
parser, one catalogue of tensor records, one group resolver made of small validators and
one transport exporter.  There is no CPU matmul: arithmetic runs on the GPU through the C ABI.
"""
import json
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

HEADER_LIMIT = 8_000_000          # bytes of JSON a file may carry
MAX_RANK = 8
MULTIPLIER = {"3inst": 0, "mcg": 0xCBAC1FED, "mul1": 0x83DCD12D}
CODEBOOK_ORDER = ("3inst", "mcg", "mul1")      # value of the C enum
RATES = frozenset((1, 2, 3, 4, 5, 6, 7, 8, 1.5, 2.5, 3.5))
I16, I32, F16, F32 = (np.dtype(code) for code in ("<i2", "<i4", "<f2", "<f4"))
NUMPY_OF = {"I16": I16, "I32": I32, "F16": F16, "F32": F32}
BITS_OF = {"BF16": np.dtype("<u2")}            # NumPy has no bfloat16: bit patterns only
# transport order and element type of each region
REGIONS = (("trellis", I16), ("suh", F16), ("svh", F16), ("bias", F32))


def _fail(message):
    raise ValueError(message)


def _aligned128(begin, end, limit):
    return (type(begin) is int and type(end) is int and 0 <= begin < end <= limit
            and begin % 128 == 0 and end % 128 == 0)


# ---- file level ------------------------------------------------------------------------
@dataclass(frozen=True)
class _Record:
    """One entry of the JSON catalogue, checked against the file size."""
    name: str
    code: str
    shape: tuple
    begin: int
    end: int

    @property
    def nbytes(self):
        return self.end - self.begin


def _object_without_repeats(pairs):
    seen = {}
    for key, value in pairs:
        if key in seen:
            _fail(f"Duplicate JSON key: {key}")
        seen[key] = value
    return seen


def _read_catalogue(path, file_bytes):
    """(header dict, byte offset of the payload area)."""
    with path.open("rb") as stream:
        prefix = stream.read(8)
        if len(prefix) < 8:
            _fail("Truncated safetensors header length")
        (length,) = struct.unpack("<Q", prefix)
        if length < 2 or length > HEADER_LIMIT or length > file_bytes - 8:
            _fail("Invalid or oversized safetensors header")
        text = stream.read(length)
    header = json.loads(text, object_pairs_hook=_object_without_repeats)
    if not isinstance(header, dict):
        _fail("Safetensors header must be an object")
    return header, 8 + length


class SafetensorsFile:
    """Selected tensors of one safetensors file as read-only memory maps; nothing is read
    until a tensor is asked for."""

    def __init__(self, path):
        self.path = Path(path)
        self.file_bytes = self.path.stat().st_size
        self.header, self.data_offset = _read_catalogue(self.path, self.file_bytes)

    # -- catalogue ----------------------------------------------------------------------
    def _record(self, name, known):
        entry = self.header.get(name)
        if not isinstance(entry, dict) or entry.get("dtype") not in known:
            _fail(f"Missing tensor or unsupported dtype: {name}")
        shape, span = entry.get("shape"), entry.get("data_offsets")
        shape_ok = (isinstance(shape, list) and len(shape) <= MAX_RANK
                    and all(type(d) is int and d >= 0 for d in shape))
        span_ok = isinstance(span, list) and len(span) == 2 and all(type(v) is int for v in span)
        if not (shape_ok and span_ok):
            _fail(f"Invalid tensor shape or offsets: {name}")
        record = _Record(name, entry["dtype"], tuple(shape), span[0], span[1])
        payload = self.file_bytes - self.data_offset
        if record.begin < 0 or record.end < record.begin or record.end > payload:
            _fail(f"Tensor range exceeds file: {name}")
        elements = 1
        for d in record.shape:
            elements *= d
        if elements * known[record.code].itemsize != record.nbytes:
            _fail(f"Tensor size does not match shape/dtype: {name}")
        return record

    def _map(self, record, dtype):
        if record.nbytes == 0:
            nothing = np.empty(record.shape, dtype=dtype)
            nothing.flags.writeable = False
            return nothing
        return np.memmap(self.path, mode="r", dtype=dtype, shape=record.shape,
                         offset=self.data_offset + record.begin)

    # -- public -------------------------------------------------------------------------
    def tensor(self, name, *, raw_bf16=False):
        known = {**NUMPY_OF, **BITS_OF} if raw_bf16 else NUMPY_OF
        record = self._record(name, known)
        return self._map(record, known[record.code])

    def tensor_float32(self, name):
        """BF16 / F16 / F32 tensor widened (exactly) to a float32 copy."""
        record = self._record(name, {**NUMPY_OF, **BITS_OF})
        values = self._map(record, {**NUMPY_OF, **BITS_OF}[record.code])
        if record.code == "BF16":
            return (values.astype(np.uint32) << 16).view(np.float32)
        if record.code not in ("F16", "F32"):
            _fail(f"Not a floating tensor: {name}")
        return np.asarray(values, dtype=np.float32)

    def exl3(self, prefix):
        return load_exl3(self, prefix)


# ---- one quantised linear ---------------------------------------------------------------
class _Transport:
    """Byte layout of the regions in the equivalent single blob: each region starts on a
    four-byte boundary, in REGIONS order; an absent bias has offset 0 and size 0."""

    def __init__(self, tensor):
        # The reference keeps 1.5 / 2.5 / 3.5 off its GPU transport (container.py:152-153); this
        # runtime decodes them on the device (mul1 only), so bits_x2 may be odd for mul1.
        if float(tensor.bits) != int(tensor.bits) and tensor.codebook != "mul1":
            _fail("GPU transport carries half-integer bitrates for mul1 only")
        self.fields = {"rows": tensor.output_size, "columns": tensor.input_size,
                       "bits_x2": int(2 * float(tensor.bits)), "codebook": CODEBOOK_ORDER.index(tensor.codebook),
                       "marker": MULTIPLIER[tensor.codebook], "transport_version": 1}
        self.members = []          # (name, source array, element dtype, offset, nbytes)
        cursor = 0
        for name, dtype in REGIONS:
            source = getattr(tensor, name)
            if source is None:
                self.fields[name + "_offset"] = self.fields[name + "_bytes"] = 0
                continue
            source = np.asarray(source)
            cursor = (cursor + 3) & ~3
            nbytes = source.size * dtype.itemsize
            self.fields[name + "_offset"], self.fields[name + "_bytes"] = cursor, nbytes
            self.members.append((name, source, dtype, cursor, nbytes))
            cursor += nbytes
        self.total = cursor

    def write(self, view):
        """Pack every member into `view` (uint8, writable); gaps between members become zero."""
        filled = 0
        for _, source, dtype, offset, nbytes in self.members:
            view[filled:offset] = 0
            window = np.ndarray(source.shape, dtype=dtype, buffer=view, offset=offset)
            np.copyto(window, source, casting="unsafe")
            filled = offset + nbytes


@dataclass(frozen=True)
class Exl3Tensor:
    """One EXL3 group with folded scales; the logical matrix Q is [input, output]."""
    trellis: np.ndarray
    suh: np.ndarray
    svh: np.ndarray
    bits: float
    codebook: str
    bias: "np.ndarray | None"
    source: str
    prefix: str

    @property
    def input_size(self):
        return 16 * self.trellis.shape[0]

    @property
    def output_size(self):
        return 16 * self.trellis.shape[1]

    def _with(self, label, **changed):
        fields = dict(trellis=self.trellis, suh=self.suh, svh=self.svh, bits=self.bits, codebook=self.codebook,
                      bias=self.bias, source=self.source, prefix=self.prefix + label)
        fields.update(changed)
        return Exl3Tensor(**fields)

    def slice_outputs(self, begin, end):
        """Column-parallel shard: whole H128 output blocks [begin, end).  The tiles stay a
        strided view; they are packed when the shard is exported."""
        if not _aligned128(begin, end, self.output_size):
            _fail("Output partitions must be nonempty, in range and H128 aligned")
        return self._with(f"[{begin}:{end}]", trellis=self.trellis[:, begin // 16:end // 16],
                          svh=self.svh[begin:end], bias=None if self.bias is None else self.bias[begin:end])

    def slice_inputs(self, begin, end, *, include_bias):
        """Row-parallel shard: whole H128 input blocks [begin, end).  The caller sums the rank
        outputs, so the bias must ride on exactly one of them: say which, explicitly."""
        if not _aligned128(begin, end, self.input_size):
            _fail("Input partitions must be nonempty, in range and H128 aligned")
        if include_bias is not True and include_bias is not False:
            _fail("include_bias must be an explicit bool")
        return self._with(f"[K{begin}:{end}]", trellis=self.trellis[begin // 16:end // 16],
                          suh=self.suh[begin:end], bias=self.bias if include_bias else None)

    # -- export -------------------------------------------------------------------------
    def transport_regions(self):
        """({region: read-only byte view or None}, metadata fields).  An array that is already
        contiguous little-endian is borrowed as it is (zero copy from the map); anything else
        -- the strided tiles of an output shard -- is packed, that region only."""
        plan = _Transport(self)
        views = {name: None for name, _ in REGIONS}
        for name, source, dtype, _, _ in plan.members:
            views[name] = memoryview(np.ascontiguousarray(source, dtype=dtype)).cast("B").toreadonly()
        return views, plan.fields

    def transport_buffer(self, destination=None):
        """The regions packed into one buffer: a fresh bytearray, or the caller's writable
        C-contiguous buffer (the used prefix comes back as a view; the tail is untouched)."""
        plan = _Transport(self)
        if destination is None:
            fresh = bytearray(plan.total)
            plan.write(np.frombuffer(fresh, dtype=np.uint8))
            return fresh, plan.fields
        try:
            raw = memoryview(destination)
        except TypeError as error:
            raise ValueError("Destination must expose a writable contiguous buffer") from error
        if raw.readonly or not raw.c_contiguous:
            _fail("Destination must be writable and C-contiguous")
        raw = raw.cast("B")
        if raw.nbytes < plan.total:
            _fail("Destination is too small for the transport")
        target = np.frombuffer(raw, dtype=np.uint8)
        for _, source, _, _, _ in plan.members:
            if np.may_share_memory(target, source):
                _fail("Destination must not overlap transport source arrays")
        plan.write(target)
        return raw[:plan.total], plan.fields

    def transport_blob(self):
        packed, fields = self.transport_buffer()
        return bytes(packed), fields

    def prepare(self, context, stream=None):
        """Upload through strix_weights_prepare_parts; returns runtime.Weights."""
        return context.prepare(self, stream)


# ---- group resolver ------------------------------------------------------------------------
def _check_tiles(tiles):
    if tiles.dtype != I16 or tiles.ndim != 3 or 0 in tiles.shape:
        _fail("EXL3 trellis must be nonempty I16 [I/16,O/16,words]")
    rate = tiles.shape[2] / 16
    if rate not in RATES:
        _fail("Unsupported EXL3 bitrate")
    inputs, outputs = 16 * tiles.shape[0], 16 * tiles.shape[1]
    if inputs % 128 or outputs % 128:
        _fail("Complete EXL3 linear requires I/O multiples of 128")
    return rate, inputs, outputs


def _check_scale(label, values, length):
    if values.dtype != F16 or values.shape != (length,) or not bool(np.isfinite(values).all()):
        _fail(f"Invalid folded F16 scale vector: {label}")


def _resolve_codebook(file, prefix, taken):
    present = [kind for kind in ("mul1", "mcg") if f"{prefix}.{kind}" in file.header]
    if len(present) == 2:
        _fail("Simultaneous mul1/mcg markers")
    if not present:
        return "3inst"
    kind = present[0]
    word = file.tensor(f"{prefix}.{kind}")
    taken[f"{prefix}.{kind}"] = word
    if word.size:  # an empty marker is the historical form: the name alone selects the codebook
        exact = word.dtype == I32 and word.size == 1
        if not exact or (int(word.reshape(-1)[0]) & 0xFFFFFFFF) != MULTIPLIER[kind]:
            _fail("Unsupported EXL3 codebook marker")
    return kind


def _resolve_bias(file, prefix, outputs, taken):
    name = prefix + ".bias"
    if name not in file.header:
        return None
    stored = file.tensor(name)
    taken[name] = stored
    if stored.dtype.kind != "f" or stored.shape != (outputs,) or not bool(np.isfinite(stored).all()):
        _fail("Invalid bias vector")
    widened = stored.astype(np.float32, copy=False)  # F32 stays mapped, F16 is converted once
    widened.flags.writeable = False
    return widened


def _require_disjoint(file, taken):
    spans = sorted(tuple(file.header[name]["data_offsets"]) for name, array in taken.items() if array.nbytes)
    for (_, left_end), (right_begin, _) in zip(spans, spans[1:]):
        if left_end > right_begin:
            _fail("Overlapping selected EXL3 tensor ranges")


def load_exl3(file, prefix):
    """Map the group `prefix`.trellis / .suh / .svh with its optional .mul1 | .mcg marker and
    .bias.  Groups that carry external out_scales are refused: their scale contract differs."""
    if not isinstance(file, SafetensorsFile):
        file = SafetensorsFile(file)
    if not isinstance(prefix, str) or prefix == "":
        _fail("A nonempty tensor prefix is required")
    if prefix + ".out_scales" in file.header:
        _fail("External out_scales requires an explicit scale contract")
    taken = {prefix + suffix: file.tensor(prefix + suffix) for suffix in (".trellis", ".suh", ".svh")}
    tiles, suh, svh = taken.values()
    rate, inputs, outputs = _check_tiles(tiles)
    _check_scale("suh", suh, inputs)
    _check_scale("svh", svh, outputs)
    codebook = _resolve_codebook(file, prefix, taken)
    if rate != int(rate) and codebook != "mul1":
        _fail("Half-integer EXL3 rates require mul1")
    bias = _resolve_bias(file, prefix, outputs, taken)
    _require_disjoint(file, taken)
    return Exl3Tensor(tiles, suh, svh, rate, codebook, bias, str(file.path), prefix)
