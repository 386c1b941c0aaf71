"""EXL3 tensor groups from local safetensors files, mapped without loading the shard,
and their export as the transport regions that strix_weights_prepare_parts consumes.

Mirrors the operator surface of the reference's python/strix_trellis/container.py
(SafetensorsFile :30-89, Exl3Tensor :92-235, load_exl3 :238-288): same names, same
argument meaning, same ValueError behaviour, so code written against the reference
loader runs unchanged.  Decoding/matmul on the CPU is NOT offered here: `matmul` runs on
the GPU through the C ABI.
"""
import json
import math
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_DTYPES = {"I16": "<i2", "I32": "<i4", "F16": "<f2", "F32": "<f4"}
_RAW_DTYPES = {"BF16": "<u2"}  # no NumPy bfloat16: raw bit patterns
_MARKERS = {"3inst": 0, "mcg": 0xCBAC1FED, "mul1": 0x83DCD12D}
_RATES = (1, 2, 3, 4, 5, 6, 7, 8, 1.5, 2.5, 3.5)
_PARTS = (("trellis", np.dtype("<i2")), ("suh", np.dtype("<f2")), ("svh", np.dtype("<f2")),
          ("bias", np.dtype("<f4")))


def _no_duplicates(pairs):
    out = {}
    for key, value in pairs:
        if key in out:
            raise ValueError(f"Duplicate JSON key: {key}")
        out[key] = value
    return out


class SafetensorsFile:
    """Read-only view of selected tensors of one safetensors file (memory mapped)."""

    def __init__(self, path):
        self.path = Path(path)
        self.file_bytes = self.path.stat().st_size
        with self.path.open("rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise ValueError("Truncated safetensors header length")
            n = struct.unpack("<Q", head)[0]
            if not 2 <= n <= min(8_000_000, self.file_bytes - 8):
                raise ValueError("Invalid or oversized safetensors header")
            self.header = json.loads(f.read(n), object_pairs_hook=_no_duplicates)
        if not isinstance(self.header, dict):
            raise ValueError("Safetensors header must be an object")
        self.data_offset = 8 + n

    def tensor(self, name, *, raw_bf16=False):
        info = self.header.get(name)
        dtypes = {**_DTYPES, **_RAW_DTYPES} if raw_bf16 else _DTYPES
        if not isinstance(info, dict) or info.get("dtype") not in dtypes:
            raise ValueError(f"Missing tensor or unsupported dtype: {name}")
        shape, offsets = info.get("shape"), info.get("data_offsets")
        if (not isinstance(shape, list) or len(shape) > 8 or any(type(x) is not int or x < 0 for x in shape)
                or not isinstance(offsets, list) or len(offsets) != 2 or any(type(x) is not int for x in offsets)):
            raise ValueError(f"Invalid tensor shape or offsets: {name}")
        begin, end = offsets
        dtype = np.dtype(dtypes[info["dtype"]])
        if not 0 <= begin <= end <= self.file_bytes - self.data_offset:
            raise ValueError(f"Tensor range exceeds file: {name}")
        if math.prod(shape) * dtype.itemsize != end - begin:
            raise ValueError(f"Tensor size does not match shape/dtype: {name}")
        if begin == end:
            empty = np.empty(shape, dtype=dtype)
            empty.flags.writeable = False
            return empty
        return np.memmap(self.path, mode="r", dtype=dtype, offset=self.data_offset + begin, shape=tuple(shape))

    def tensor_float32(self, name):
        info = self.header.get(name)
        kind = info.get("dtype") if isinstance(info, dict) else None
        raw = self.tensor(name, raw_bf16=True)
        if kind == "BF16":
            return (raw.astype(np.uint32) << 16).view(np.float32)
        if kind in ("F16", "F32"):
            return np.asarray(raw, dtype=np.float32)
        raise ValueError(f"Not a floating tensor: {name}")

    def exl3(self, prefix):
        return load_exl3(self, prefix)


@dataclass(frozen=True)
class Exl3Tensor:
    """Folded-scale EXL3 group; logical Q is [input, output]."""
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
        return self.trellis.shape[0] * 16

    @property
    def output_size(self):
        return self.trellis.shape[1] * 16

    def slice_outputs(self, begin, end):
        """H128-aligned output partition (column-parallel shard); the tile stride is
        repacked when the slice is exported."""
        if (type(begin) is not int or type(end) is not int or not 0 <= begin < end <= self.output_size
                or begin % 128 or end % 128):
            raise ValueError("Output partitions must be nonempty, in range and H128 aligned")
        return Exl3Tensor(self.trellis[:, begin // 16:end // 16, :], self.suh, self.svh[begin:end], self.bits,
                          self.codebook, None if self.bias is None else self.bias[begin:end], self.source,
                          self.prefix + f"[{begin}:{end}]")

    def slice_inputs(self, begin, end, *, include_bias):
        """H128-aligned input partition (row-parallel shard).  Rank outputs are summed by
        the caller; exactly one rank carries the bias."""
        if (type(begin) is not int or type(end) is not int or not 0 <= begin < end <= self.input_size
                or begin % 128 or end % 128):
            raise ValueError("Input partitions must be nonempty, in range and H128 aligned")
        if type(include_bias) is not bool:
            raise ValueError("include_bias must be an explicit bool")
        return Exl3Tensor(self.trellis[begin // 16:end // 16, :, :], self.suh[begin:end], self.svh, self.bits,
                          self.codebook, self.bias if include_bias else None, self.source,
                          self.prefix + f"[K{begin}:{end}]")

    def _layout(self):
        if not float(self.bits).is_integer():
            raise ValueError("GPU transport v1 supports integer bitrates only")
        meta = dict(rows=self.output_size, columns=self.input_size, bits_x2=int(self.bits) * 2,
                    codebook=("3inst", "mcg", "mul1").index(self.codebook), marker=_MARKERS[self.codebook],
                    transport_version=1)
        arrays, size = [], 0
        for name, dtype in _PARTS:
            values = getattr(self, name)
            if values is None:
                meta[name + "_offset"] = meta[name + "_bytes"] = 0
                continue
            values = np.asarray(values)
            size += -size % 4
            meta[name + "_offset"] = size
            meta[name + "_bytes"] = values.size * dtype.itemsize
            size += meta[name + "_bytes"]
            arrays.append((name, values, dtype))
        return arrays, meta, size

    def transport_regions(self):
        """(read-only byte views, metadata).  Contiguous little-endian arrays are borrowed
        (zero copy from the memory map); an output slice repacks only its trellis."""
        arrays, meta, _ = self._layout()
        regions = dict.fromkeys(name for name, _ in _PARTS)
        for name, values, dtype in arrays:
            regions[name] = memoryview(np.ascontiguousarray(values, dtype=dtype)).cast("B").toreadonly()
        return regions, meta

    def transport_buffer(self, destination=None):
        arrays, meta, size = self._layout()
        owned = destination is None
        if owned:
            destination = bytearray(size)
        try:
            view = memoryview(destination)
        except TypeError as error:
            raise ValueError("Destination must expose a writable contiguous buffer") from error
        if view.readonly or not view.c_contiguous:
            raise ValueError("Destination must be writable and C-contiguous")
        view = view.cast("B")
        if view.nbytes < size:
            raise ValueError("Destination is too small for the transport")
        if not owned:
            target = np.frombuffer(view, dtype=np.uint8)
            if any(np.may_share_memory(target, values) for _, values, _ in arrays):
                raise ValueError("Destination must not overlap transport source arrays")
        end = 0
        for name, values, dtype in arrays:
            offset, length = meta[name + "_offset"], meta[name + "_bytes"]
            if offset > end:
                view[end:offset] = b"\0" * (offset - end)
            np.copyto(np.ndarray(values.shape, dtype=dtype, buffer=view, offset=offset), values, casting="unsafe")
            end = offset + length
        return (destination if owned else view[:size]), meta

    def transport_blob(self):
        data, meta = self.transport_buffer()
        return bytes(data), meta

    def prepare(self, context, stream=None):
        """Upload to the GPU through strix_weights_prepare_parts; returns runtime.Weights."""
        return context.prepare(self, stream)


def load_exl3(file, prefix):
    """Map one EXL3 group (`prefix`.trellis/.suh/.svh [+ .mul1/.mcg marker, .bias])."""
    file = file if isinstance(file, SafetensorsFile) else SafetensorsFile(file)
    if not isinstance(prefix, str) or not prefix:
        raise ValueError("A nonempty tensor prefix is required")
    if prefix + ".out_scales" in file.header:
        raise ValueError("External out_scales requires an explicit scale contract")
    names = [prefix + s for s in (".trellis", ".suh", ".svh")]
    chosen = {n: file.tensor(n) for n in names}
    trellis, suh, svh = (chosen[n] for n in names)
    if trellis.dtype != np.dtype("<i2") or trellis.ndim != 3 or not all(trellis.shape):
        raise ValueError("EXL3 trellis must be nonempty I16 [I/16,O/16,words]")
    bits = trellis.shape[-1] / 16
    if bits not in _RATES:
        raise ValueError("Unsupported EXL3 bitrate")
    inputs, outputs = trellis.shape[0] * 16, trellis.shape[1] * 16
    if inputs % 128 or outputs % 128:
        raise ValueError("Complete EXL3 linear requires I/O multiples of 128")
    for name, values, size in (("suh", suh, inputs), ("svh", svh, outputs)):
        if values.dtype != np.dtype("<f2") or values.shape != (size,) or not np.isfinite(values).all():
            raise ValueError(f"Invalid folded F16 scale vector: {name}")
    markers = [m for m in ("mul1", "mcg") if prefix + "." + m in file.header]
    if len(markers) > 1:
        raise ValueError("Simultaneous mul1/mcg markers")
    codebook = markers[0] if markers else "3inst"
    if markers:
        name = prefix + "." + codebook
        marker = file.tensor(name)
        chosen[name] = marker
        if marker.size and (marker.dtype != np.dtype("<i4") or marker.size != 1
                            or int(marker.reshape(-1)[0]) & 0xFFFFFFFF != _MARKERS[codebook]):
            raise ValueError("Unsupported EXL3 codebook marker")
    if bits % 1 and codebook != "mul1":
        raise ValueError("Half-integer EXL3 rates require mul1")
    bias = None
    if prefix + ".bias" in file.header:
        name = prefix + ".bias"
        raw = file.tensor(name)
        chosen[name] = raw
        if raw.dtype.kind != "f" or raw.shape != (outputs,) or not np.isfinite(raw).all():
            raise ValueError("Invalid bias vector")
        bias = raw.astype(np.float32, copy=False)
        bias.flags.writeable = False
    spans = sorted(file.header[n]["data_offsets"] for n, v in chosen.items() if v.nbytes)
    if any(a[1] > b[0] for a, b in zip(spans, spans[1:])):
        raise ValueError("Overlapping selected EXL3 tensor ranges")
    return Exl3Tensor(trellis, suh, svh, bits, codebook, bias, str(file.path), prefix)
