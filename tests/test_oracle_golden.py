"""Pins the CPU oracles (NumPy and C) to the reference: its own known-answer
vectors, and stage outputs produced by running its Python package
(tests/golden/make_golden.py)."""
import hashlib
import json

import numpy as np
import pytest

from oracle import c_oracle, trellis_ref as ref
from strix_trellis_b200 import synthetic


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# reference tests/test_numerics.py:74-87 (docs/NUMERICS.md:136-140)
CODEBOOK_SHA = {
    "3inst": "ad88de2dcff5bb05fff2faec37cceceb43aa1c2e8203f9d81a6fbd6dd3393eea",
    "mcg": "95383563929baa9d1ae5de0be22490284382673620bdd85929feea7bdbef04a9",
    "mul1": "bc48d02cb1c14939dc47b90f870dd689d63e3b1ab69a157e65538db68677a6c8",
}
# reference tests/test_reference.py:83-95
SPOT_STATES = [0, 1, 2, 255, 256, 32767, 32768, 65535]
SPOT_BITS = {
    "mul1": [0xc2e8, 0x3921, 0xb72d, 0x3ab3, 0xb3db, 0x3fca, 0xbaf2, 0xb936],
    "mcg": [0x3f60, 0x304e, 0xba13, 0xbd26, 0xbaf0, 0x4172, 0xb915, 0x3acd],
    "3inst": [0x3a25, 0xbb5b, 0x3b74, 0x3cd1, 0x3c3f, 0xba96, 0xb7f8, 0xb110],
}


@pytest.mark.parametrize("name", ref.CODEBOOK_NAMES)
def test_codebook_hash_and_spot_values(name):
    table = ref.codebook_table(name)
    assert sha(table.astype("<f2")) == CODEBOOK_SHA[name]
    assert list(table[SPOT_STATES].view(np.uint16)) == SPOT_BITS[name]
    ctable = c_oracle.codebook_table(ref.CODEBOOK_NAMES.index(name))
    assert ctable.tobytes() == table.tobytes()


def bit_serial_states(tile, k):
    """Independent shift register over the physical bytes (the approach of
    reference tests/test_reference.py:17-36, rewritten)."""
    raw = np.asarray(tile, dtype="<u2").tobytes()
    bits = []
    for off in range(0, len(raw), 4):
        word = int.from_bytes(raw[off:off + 4], "little")
        bits.extend((word >> (31 - b)) & 1 for b in range(32))
    state = 0
    for b in bits[-16:]:
        state = (state << 1) | b
    out, cursor = [], 0
    for i in range(256):
        width = int(k) + (i % 2 if k % 1 else 0)
        for b in bits[cursor:cursor + width]:
            state = ((state << 1) | b) & 0xFFFF
        out.append(state)
        cursor += width
    return np.array(out, dtype=np.uint16)


@pytest.mark.parametrize("k", [1, 2, 3, 4, 5, 6, 7, 8, 1.5, 2.5, 3.5])
def test_ring_states_against_shift_register(k):
    rng = np.random.default_rng(9823)
    words = rng.integers(0, 65536, (3, int(16 * k)), dtype=np.uint16)
    got = ref.ring_states(words, k)
    for i in range(3):
        np.testing.assert_array_equal(got[i], bit_serial_states(words[i], k))
        if float(k).is_integer():
            np.testing.assert_array_equal(c_oracle.unpack_states(words[i], int(k)), got[i])
    np.testing.assert_array_equal(got, ref.ring_states(words.view(np.int16), k))


def test_ring_wrap_and_word_order():
    # reference tests/test_reference.py:53-62
    words = np.zeros(16, dtype=np.uint16)
    words[1] = 0x8000
    states = ref.ring_states(words, 1)
    np.testing.assert_array_equal(states[:16], 1 << np.arange(16))
    assert states[16] == 0
    words[:] = 0
    words[-2] = 1
    assert ref.ring_states(words, 1)[0] == 2


def test_fragment_coordinates():
    # reference tests/test_reference.py:64-81, docs/FORMAT.md:61-66
    words = np.random.default_rng(12).integers(0, 65536, (1, 1, 128), dtype=np.uint16)
    values = ref.states_to_values(ref.ring_states(words[0, 0], 8))
    tile = ref.dequantize(words, 8)
    for lane in range(32):
        for frag in range(8):
            row = 2 * (lane % 4) + frag % 2 + 8 * ((frag // 2) % 2)
            col = lane // 4 + 8 * (frag // 4)
            assert tile[row, col] == values[8 * lane + frag]


def test_prescale_double_rounding_regression():
    # reference tests/test_numerics.py:46-54
    x = np.zeros(128, dtype=np.float32)
    s = np.ones(128, dtype=np.float16)
    x[0] = np.float32(0.2001299113035202)
    s[0] = np.float16(0.02642822265625)
    assert int(ref.input_stages(x[None], s)["scaled_fp16"].view(np.uint16)[0, 0]) == 0x1D6A
    assert int(c_oracle.input_stages(x[None], s)["scaled_fp16"].view(np.uint16)[0, 0]) == 0x1D6A


def test_hadamard_impulses():
    # reference tests/test_numerics.py:89-96
    x = np.eye(128, dtype=np.float32)
    parity = np.array([[1 if bin(i & j).count("1") % 2 == 0 else -1 for j in range(128)]
                       for i in range(128)], dtype=np.float32)
    np.testing.assert_array_equal(ref.hadamard128_fp32(x), parity * np.float32(1 / np.sqrt(128)))


def test_core_fixed_order():
    # reference tests/test_numerics.py:115-126
    a = np.array([[2048, 1, 2048], [1, -2, 0.5]], dtype=np.float16)
    q = np.array([[2048, 2], [0.125, -3], [-2048, 4]], dtype=np.float16)
    got = ref.core_dot(a, q)
    assert got[0, 0] == 0
    np.testing.assert_array_equal(c_oracle.core_dot(a, q), got)


def _grid(golden_dir):
    meta = json.loads((golden_dir / "grid.json").read_text())
    return meta, np.load(golden_dir / "grid_ref.npz")


def test_grid_numpy_oracle_matches_reference_stages(golden_dir):
    meta, outs = _grid(golden_dir)
    for case in meta["cases"]:
        layer, x, old, seed = synthetic.grid_case(case["codebook"], case["bits"], case["wide"], meta["rows"])
        assert seed == case["seed"]
        blob = np.concatenate([layer.trellis.ravel().view(np.uint8), layer.suh.view(np.uint8),
                               layer.svh.view(np.uint8), x.ravel().view(np.uint8), old.ravel().view(np.uint8)])
        assert sha(blob) == case["inputs_sha"], case["name"]
        st = ref.linear_stages(x, layer.trellis, layer.suh, layer.svh, layer.bits, layer.codebook, layer.bias)
        assert sha(st["rotated_fp16"]) == case["q"], case["name"]
        assert sha(st["scaled_fp16"]) == case["scaled"]
        assert sha(st["input_hadamard_fp32"]) == case["inh"]
        assert sha(st["core_input_fp16"]) == case["a"]
        assert sha(st["core_fp32"]) == case["core"]
        assert sha(st["output_hadamard_fp32"]) == case["out_h"]
        assert sha(st["output_fp32"]) == case["ref"]
        assert st["output_fp32"].tobytes() == outs[case["name"]].tobytes()


def test_grid_c_oracle_matches_reference_stages(golden_dir):
    meta, outs = _grid(golden_dir)
    for case in meta["cases"]:
        layer, x, old, _ = synthetic.grid_case(case["codebook"], case["bits"], case["wide"], meta["rows"])
        assert sha(c_oracle.dequantize(layer.trellis, layer.bits, case["codebook"])) == case["q"]
        st = c_oracle.input_stages(x, layer.suh)
        assert sha(st["scaled_fp16"]) == case["scaled"]
        assert sha(st["input_hadamard_fp32"]) == case["inh"]
        assert sha(st["core_input_fp16"]) == case["a"]
        out, core = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, layer.bits,
                                    case["codebook"], x, return_core=True)
        assert sha(core) == case["core"]
        assert sha(out) == case["ref"], case["name"]
        for alpha, beta in [(-0.75, 0.25), (0.0, -0.5), (1.0, -0.0)]:
            want = ref.apply_alpha_beta(outs[case["name"]], alpha, beta, old)
            got = c_oracle.linear(layer.trellis, layer.suh, layer.svh, layer.bias, layer.bits,
                                  case["codebook"], x, alpha, beta, old)
            assert got.tobytes() == want.tobytes()


def test_config1_c_oracle(golden_dir):
    meta = json.loads((golden_dir / "config1.json").read_text())
    gold = np.load(golden_dir / "config1.npz")
    layer = synthetic.make_layer(4096, 4096, 4, seed=meta["seed"])
    x = synthetic.make_activations(1, 4096, seed=meta["x_seed"])
    assert sha(layer.trellis) == meta["trellis_sha"] and sha(x) == meta["x_sha"]
    assert sha(c_oracle.dequantize(layer.trellis, 4, 2)) == meta["q"]
    out, core = c_oracle.linear(layer.trellis, layer.suh, layer.svh, None, 4, 2, x, return_core=True)
    assert sha(core) == meta["core"] and sha(out) == meta["ref"]
    assert out.tobytes() == gold["ref"].tobytes()


def test_half_rates(golden_dir):
    meta = json.loads((golden_dir / "half_rates.json").read_text())
    rng = synthetic.rng_for(synthetic.BASE_SEED + 50)
    for rate in (1.5, 2.5, 3.5):
        t = rng.integers(0, 65536, (8, 8, int(16 * rate)), dtype=np.uint16)
        assert sha(t) == meta[str(rate)]["trellis_sha"]
        assert sha(ref.ring_states(t, rate)) == meta[str(rate)]["states"]
        assert sha(ref.dequantize(t, rate, "mul1")) == meta[str(rate)]["q"]


def test_reference_host_decoder_agrees_when_built():
    host = c_oracle.reference_host_decoder()
    if host is None:
        pytest.skip("oracle/_ref not built here (needs the reference tree)")
    rng = np.random.default_rng(5)
    for cb in range(3):
        table = c_oracle.codebook_table(cb).view(np.uint16)
        for s in rng.integers(0, 65536, 2000):
            assert host.ref_host_codebook(int(s), cb) == table[s]
    for k in range(1, 9):
        tile = rng.integers(0, 65536, 16 * k, dtype=np.uint16)
        words = np.ascontiguousarray(tile).view(np.uint32)
        states = c_oracle.unpack_states(tile, k)
        for i in range(256):
            assert host.ref_host_state(words.ctypes.data, k, i) == states[i]


def test_moe_oracle_matches_reference_composition(golden_dir):
    gold = np.load(golden_dir / "moe_small.npz")
    hidden_dim, inter, n_exp, top_k, tokens = 256, 128, 8, 3, 4
    experts = {}
    for e in range(n_exp):
        bits = {"gate": 2 + e % 2, "up": 3 if e % 3 == 0 else 2, "down": 2 if e % 3 == 1 else 3}
        layers = {
            "gate": synthetic.make_layer(hidden_dim, inter, bits["gate"], synthetic.BASE_SEED + 700 + 3 * e, sigma=0.5, bias=True),
            "up": synthetic.make_layer(hidden_dim, inter, bits["up"], synthetic.BASE_SEED + 701 + 3 * e, sigma=0.5),
            "down": synthetic.make_layer(inter, hidden_dim, bits["down"], synthetic.BASE_SEED + 702 + 3 * e, sigma=0.5, bias=True)}
        experts[e] = {k: (w.trellis, w.suh, w.svh, w.bits, w.codebook, w.bias) for k, w in layers.items()}
    x = synthetic.make_activations(tokens, hidden_dim, seed=synthetic.BASE_SEED + 790)
    y, hidden = ref.moe_block(x, experts, gold["ids"], gold["scores"])
    assert y.tobytes() == gold["y"].tobytes()
    for (r, s), h in hidden.items():
        assert h.tobytes() == gold["hidden"][r, s].tobytes()
    assert (1, 2) not in hidden  # zero score skipped


def test_tp_slices_recombine(golden_dir):
    gold = np.load(golden_dir / "tp_small.npz")
    layer = synthetic.make_layer(512, 384, 5, seed=synthetic.BASE_SEED + 60, bias=True)
    x = synthetic.make_activations(3, 512, seed=synthetic.BASE_SEED + 61)
    full = ref.linear_stages(x, layer.trellis, layer.suh, layer.svh, 5, "mul1", layer.bias)["output_fp32"]
    assert full.tobytes() == gold["full"].tobytes()
    for parts in (2, 3):
        pieces = []
        for r, (b0, b1) in enumerate(ref.h128_bounds(384, parts)):
            out = ref.linear_stages(x, layer.trellis[:, b0 // 16:b1 // 16], layer.suh, layer.svh[b0:b1],
                                    5, "mul1", layer.bias[b0:b1])["output_fp32"]
            pieces.append(out)
        # column shards are bit-identical to the same columns of the full result
        assert np.concatenate(pieces, axis=1).tobytes() == full.tobytes()
    for parts in (2, 4):
        total = np.zeros_like(full)
        for r, (a0, a1) in enumerate(ref.h128_bounds(512, parts)):
            out = ref.linear_stages(x[:, a0:a1], layer.trellis[a0 // 16:a1 // 16], layer.suh[a0:a1],
                                    layer.svh, 5, "mul1", layer.bias if r == 0 else None)["output_fp32"]
            assert out.tobytes() == gold[f"in{parts}_{r}"].tobytes()
            total += out
        assert np.abs(total - full).max() <= 5e-4 * max(1.0, np.abs(full).max())
