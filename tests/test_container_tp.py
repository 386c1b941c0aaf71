"""Loader and partition host logic (no GPU): the safetensors reader's acceptance and
rejection rules (reference tests/test_container.py), transport export, N-rank partitions,
and the world_size-2 recombination collectives over gloo."""
import hashlib
import json
import os
import struct

import numpy as np
import pytest

from strix_trellis_b200 import container, synthetic, tp

NAMES = {"int16": "I16", "int32": "I32", "float16": "F16", "float32": "F32"}


def tensors(bits=3, marker="mul1"):
    rng = np.random.default_rng(73)
    out = {"projection.trellis": rng.integers(-32768, 32768, (8, 16, 16 * bits), dtype=np.int16),
           "projection.suh": np.linspace(-1, 1, 128, dtype=np.float16),
           "projection.svh": np.linspace(0.25, -0.5, 256, dtype=np.float16),
           "projection.bias": (np.arange(256, dtype=np.float32) / 256)}
    if marker:
        word = {"mul1": 0x83DCD12D, "mcg": 0xCBAC1FED}[marker]
        out["projection." + marker] = np.array([word], dtype=np.uint32).view(np.int32)
    return out


def write_file(path, values, mutate=None):
    data, header = bytearray(), {}
    for name, array in values.items():
        payload = array.tobytes()
        header[name] = dict(dtype=NAMES[array.dtype.name], shape=list(array.shape),
                            data_offsets=[len(data), len(data) + len(payload)])
        data.extend(payload)
    if mutate:
        mutate(header)
    raw = json.dumps(header).encode()
    raw += b" " * (-len(raw) % 8)
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + data)


def test_load_and_transport_layout(tmp_path):
    path = tmp_path / "m.safetensors"
    values = tensors()
    write_file(path, values)
    t = container.load_exl3(path, "projection")
    assert (t.input_size, t.output_size, t.bits, t.codebook) == (128, 256, 3, "mul1")
    blob, meta = t.transport_blob()
    assert meta["rows"] == 256 and meta["columns"] == 128 and meta["bits_x2"] == 6
    assert meta["marker"] == 0x83DCD12D and meta["codebook"] == 2
    for name in ("trellis", "suh", "svh", "bias"):
        off, n = meta[name + "_offset"], meta[name + "_bytes"]
        assert off % 4 == 0 and blob[off:off + n] == values["projection." + name].tobytes()
    regions, meta2 = t.transport_regions()
    assert meta2 == meta and bytes(regions["trellis"]) == values["projection.trellis"].tobytes()
    assert regions["trellis"].readonly
    # contiguous payloads are borrowed from the memory map, not copied
    assert np.shares_memory(np.frombuffer(regions["suh"], dtype=np.uint8), t.suh)


@pytest.mark.parametrize("case", ["truncated", "dup", "out_scales", "two_markers", "bad_marker", "overlap",
                                  "bad_scale", "odd_dims"])
def test_rejections(tmp_path, case):
    path = tmp_path / "m.safetensors"
    values = tensors()
    if case == "truncated":
        path.write_bytes(b"\x01\x02")
    elif case == "dup":
        raw = b'{"a":{"dtype":"F16","shape":[1],"data_offsets":[0,2]},"a":{"dtype":"F16","shape":[1],"data_offsets":[0,2]}}'
        path.write_bytes(struct.pack("<Q", len(raw)) + raw + b"\0\0")
        with pytest.raises(ValueError):
            container.SafetensorsFile(path)
        return
    elif case == "out_scales":
        values["projection.out_scales"] = np.ones(2, np.float16)
        write_file(path, values)
    elif case == "two_markers":
        values["projection.mcg"] = np.array([0xCBAC1FED], dtype=np.uint32).view(np.int32)
        write_file(path, values)
    elif case == "bad_marker":
        values["projection.mul1"] = np.array([5], dtype=np.int32)
        write_file(path, values)
    elif case == "overlap":
        def mutate(h):
            h["projection.suh"]["data_offsets"] = [0, 256]
        write_file(path, values, mutate)
    elif case == "bad_scale":
        values["projection.suh"] = values["projection.suh"].copy()
        values["projection.suh"][3] = np.inf
        write_file(path, values)
    elif case == "odd_dims":
        values["projection.trellis"] = values["projection.trellis"][:7]
        write_file(path, values)
    with pytest.raises(ValueError):
        container.load_exl3(path, "projection")


def test_slices_and_transport_match_reference_golden(golden_dir):
    gold = np.load(golden_dir / "tp_small.npz")
    layer = synthetic.make_layer(512, 384, 5, seed=synthetic.BASE_SEED + 60, bias=True)
    full = container.Exl3Tensor(layer.trellis.view(np.int16), layer.suh, layer.svh, 5, "mul1", layer.bias, "s", "w")
    for parts in (2, 3):
        for r in range(parts):
            b0, b1 = 128 * (3 * r // parts), 128 * (3 * (r + 1) // parts)
            if b1 > b0:
                blob, meta = full.slice_outputs(b0, b1).transport_blob()
                assert hashlib.sha256(blob).digest() == gold[f"out{parts}_{r}_blob_sha"].tobytes()
                assert meta["rows"] == b1 - b0
    with pytest.raises(ValueError):
        full.slice_outputs(0, 100)
    with pytest.raises(ValueError):
        full.slice_inputs(0, 128, include_bias=1)
    part = full.slice_inputs(128, 384, include_bias=False)
    assert part.bias is None and np.shares_memory(part.trellis, full.trellis) and part.svh is full.svh


def test_rank_partition_any_world():
    layer = synthetic.make_layer(1024, 129280 // 10 // 128 * 128, 2, seed=3)
    full = container.Exl3Tensor(layer.trellis.view(np.int16), layer.suh, layer.svh, 2, "mul1", None, "s", "w")
    for world in (1, 2, 4, 8):
        widths = [tp.rank_partition(full, "output", r, world).output_size for r in range(world)]
        assert sum(widths) == full.output_size and max(widths) - min(widths) <= 128
        ins = [tp.rank_partition(full, "input", r, world) for r in range(world)]
        assert sum(p.input_size for p in ins) == 1024
    assert tp.h128_bounds(129280, 8)[0] == (0, 127 * 128) and tp.h128_bounds(129280, 8)[-1][1] == 129280
    assert tp.rank_partition(full, "replicate", 1, 2) is full
    with pytest.raises(ValueError):
        tp.rank_partition(full, "output", 2, 2)
    assert [tp.expert_owner(e, 256, 8) for e in (0, 31, 32, 255)] == [0, 0, 1, 7]


def _worker(rank, world, port, tmp):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    widths = [256, 128]
    full = torch.arange(3 * 384, dtype=torch.float32).reshape(3, 384)
    off = sum(widths[:rank])
    got = tp.all_gather_columns(full[:, off:off + widths[rank]].contiguous(), widths)
    assert torch.equal(got, full)
    part = torch.full((2, 8), float(rank + 1))
    tp.all_reduce_rows(part)
    assert torch.equal(part, torch.full((2, 8), 3.0))
    dist.destroy_process_group()
    open(os.path.join(tmp, f"ok{rank}"), "w").close()


def test_recombination_collectives_world2_gloo(tmp_path):
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
