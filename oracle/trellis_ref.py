"""CPU oracle (NumPy) for the EXL3 trellis linear layer.  TEST INFRASTRUCTURE ONLY.

This module restates, in independent NumPy code, the algorithm of the reference
project's CPU contract.  It exists so that the CUDA path can be checked; nothing
in the shipped package may import it.  Only tests, the smoke check and the
benchmark's CPU-baseline leg use it.

Parity status: PINNED.  `tests/test_oracle_golden.py` checks every function
against (a) the known-answer vectors in the reference's own tests
(tests/test_reference.py:83-95 codebook spot values, tests/test_numerics.py:74-87
SHA-256 of all 65 536 codebook outputs, tests/test_numerics.py:46-54 double
rounding regression) and (b) stage-by-stage outputs produced by importing the
reference's `python/strix_trellis` package, stored under tests/golden/.

Each function cites the reference file:line it follows.
"""
import numpy as np

CODEBOOK_NAMES = ("3inst", "mcg", "mul1")
MARKERS = {"3inst": 0, "mcg": 0xCBAC1FED, "mul1": 0x83DCD12D}
_INV_SQRT128 = np.float32(1.0 / np.sqrt(128.0))


def rate_widths(k):
    """Bits consumed by each of the 256 stream positions (codec.py:12-20).

    Integer K gives K everywhere; K+1/2 alternates K, K+1 starting with K."""
    rate = float(k)
    if rate not in (1, 2, 3, 4, 5, 6, 7, 8, 1.5, 2.5, 3.5):
        raise ValueError("unsupported bitrate")
    base = int(rate)
    odd = 0 if rate == base else 1
    return np.array([base + (i & 1) * odd for i in range(256)], dtype=np.int64)


def ring_states(packed, k):
    """16-bit trellis states of every stream position (codec.py:58-85).

    `packed` is (..., 16K) 16-bit containers.  Pairs form little-endian uint32
    ring words read most-significant bit first; state i is the 16 ring bits that
    end at the cumulative width S(i), indices modulo the ring length."""
    widths = rate_widths(k)
    ring_bits = int(widths.sum())
    halves = np.asarray(packed)
    if halves.dtype.kind not in "iu" or halves.dtype.itemsize != 2:
        raise ValueError("containers must be 16-bit integers")
    if halves.shape[-1] != ring_bits // 16:
        raise ValueError("wrong container count for this rate")
    h = halves.astype(np.uint16).astype(np.uint64)  # numeric value, any byte order
    words = h[..., 0::2] | (h[..., 1::2] << np.uint64(16))
    nwords = ring_bits // 32
    ends = np.cumsum(widths)
    starts = (ends - 16) % ring_bits
    first = starts // 32
    offset = (starts % 32).astype(np.uint64)
    pair = (words[..., first % nwords] << np.uint64(32)) | words[..., (first + 1) % nwords]
    return ((pair >> (np.uint64(48) - offset)) & np.uint64(0xFFFF)).astype(np.uint16)


def _half_bits_to_units(bits):
    """Exact value of binary16 bit patterns in units of 2**-24 (int64)."""
    bits = bits.astype(np.int64)
    exponent = (bits >> 10) & 31
    fraction = bits & 1023
    magnitude = np.where(exponent == 0, fraction, (1024 + fraction) << np.maximum(exponent - 1, 0))
    return np.where(bits & 0x8000, -magnitude, magnitude)


_TABLES = {}


def codebook_table(name):
    """All 65 536 codebook outputs as float16 (codec.py:27-47, docs/FORMAT.md:73-86).

    mul1: p = s*0x83DCD12D mod 2**32, b = sum of its four bytes,
    value = RN16(((1024+b)*1774 - 1329*2048) / 2**18) (one rounding).
    3inst/mcg: p = s*89226354+64248484 or s*0xCBAC1FED, q = (p & 0x8FFF8FFF) ^
    0x3B603B60, value = RN16(half(lo16 q) + half(hi16 q)) (one rounding)."""
    if name not in CODEBOOK_NAMES:
        raise ValueError("unknown codebook")
    if name in _TABLES:
        return _TABLES[name]
    s = np.arange(65536, dtype=np.uint64)
    if name == "mul1":
        p = (s * np.uint64(0x83DCD12D)) & np.uint64(0xFFFFFFFF)
        b = sum(((p >> np.uint64(sh)) & np.uint64(255)).astype(np.int64) for sh in (0, 8, 16, 24))
        numerator = (1024 + b) * 1774 - 1329 * 2048  # exact, |.| < 2**53
        table = (numerator.astype(np.float64) / 262144.0).astype(np.float16)
    else:
        mult, add = (89226354, 64248484) if name == "3inst" else (0xCBAC1FED, 0)
        p = (s * np.uint64(mult) + np.uint64(add)) & np.uint64(0xFFFFFFFF)
        q = (p & np.uint64(0x8FFF8FFF)) ^ np.uint64(0x3B603B60)
        units = _half_bits_to_units(q & np.uint64(0xFFFF)) + _half_bits_to_units(q >> np.uint64(16))
        table = (units.astype(np.float64) / 16777216.0).astype(np.float16)
    table.flags.writeable = False
    _TABLES[name] = table
    return table


def states_to_values(states, codebook="mul1"):
    """float16 value of each state, taken modulo 2**16 (codec.py:50-55)."""
    return codebook_table(codebook)[np.asarray(states).astype(np.uint16)]


def _stream_position():
    """Stream position of logical (input row r, output column c) inside a tile
    (codec.py:94-100): ((c&7)<<5) | ((r&6)<<2) | (r&1) | ((r&8)>>2) | ((c&8)>>1)."""
    r = np.arange(16)[:, None]
    c = np.arange(16)[None, :]
    return ((c & 7) << 5) | ((r & 6) << 2) | (r & 1) | ((r & 8) >> 2) | ((c & 8) >> 1)


_POSITION = _stream_position()


def dequantize(trellis, k=None, codebook="mul1", chunk=4096):
    """[I/16, N/16, 16K] containers -> rotated weights Q [I, N] float16
    (codec.py:150-173)."""
    t = np.asarray(trellis)
    if t.ndim != 3 or 0 in t.shape:
        raise ValueError("trellis must be a nonempty rank-3 array")
    if k is None:
        k = t.shape[-1] / 16
    if float(k) % 1 and codebook != "mul1":
        raise ValueError("half-integer rates need mul1")
    flat = t.reshape(-1, t.shape[-1])
    out = np.empty((flat.shape[0], 16, 16), dtype=np.float16)
    for begin in range(0, flat.shape[0], chunk):
        values = states_to_values(ring_states(flat[begin:begin + chunk], k), codebook)
        out[begin:begin + chunk] = values[:, _POSITION]
    tiles = out.reshape(t.shape[0], t.shape[1], 16, 16)
    return tiles.transpose(0, 2, 1, 3).reshape(t.shape[0] * 16, t.shape[1] * 16)


def hadamard128_fp32(values):
    """Block-diagonal H128 on the last axis in float32 (linear.py:82-108):
    butterflies with strides 1,2,...,64, every add/sub rounded to float32,
    then ONE multiply by RN32(1/sqrt(128))."""
    data = np.array(values, dtype=np.float32, copy=True)
    if data.shape[-1] % 128:
        raise ValueError("last axis must be a multiple of 128")
    blocks = data.reshape(-1, 128)
    stride = 1
    while stride < 128:
        g = blocks.reshape(-1, 128 // (2 * stride), 2, stride)
        lo = g[:, :, 0, :].copy()
        hi = g[:, :, 1, :].copy()
        g[:, :, 0, :] = lo + hi
        g[:, :, 1, :] = lo - hi
        stride *= 2
    blocks *= _INV_SQRT128
    return blocks.reshape(data.shape)


def input_stages(x, suh):
    """x -> core input A (linear.py:111-124): RN32(x*f32(suh)) -> RN16 -> H128
    (float32) -> RN16."""
    x32 = np.asarray(x, dtype=np.float32)
    s16 = np.asarray(suh).astype(np.float16)
    scaled32 = x32 * s16.astype(np.float32)
    scaled16 = scaled32.astype(np.float16)
    had = hadamard128_fp32(scaled16.astype(np.float32))
    return {"scaled_fp32": scaled32, "scaled_fp16": scaled16,
            "input_hadamard_fp32": had, "core_input_fp16": had.astype(np.float16)}


def core_dot(a16, q16):
    """acc=+0; for i ascending: acc = RN32(acc + RN32(a_i*q_io)) (linear.py:127-143)."""
    a = np.asarray(a16, dtype=np.float16).astype(np.float32)
    q = np.asarray(q16, dtype=np.float16).astype(np.float32)
    acc = np.zeros(a.shape[:-1] + (q.shape[1],), dtype=np.float32)
    for i in range(q.shape[0]):
        acc += a[..., i, None] * q[i]
    return acc


def output_stages(core, svh, bias=None):
    """core -> Linear(x) (linear.py:146-163): H128 float32, * f32(svh), + bias."""
    had = hadamard128_fp32(np.asarray(core, dtype=np.float32))
    scaled = had * np.asarray(svh).astype(np.float16).astype(np.float32)
    out = scaled if bias is None else scaled + np.asarray(bias, dtype=np.float32)
    return {"output_hadamard_fp32": had, "scaled_output_fp32": scaled, "output_fp32": out}


def linear_stages(x, trellis, suh, svh, k=None, codebook="mul1", bias=None):
    """Every checkpoint of the staged float32 contract (linear.py:166-175)."""
    q = dequantize(trellis, k, codebook)
    st = input_stages(x, suh)
    st["rotated_fp16"] = q
    st["core_fp32"] = core_dot(st["core_input_fp16"], q)
    st.update(output_stages(st["core_fp32"], svh, bias))
    return st


def apply_alpha_beta(linear, alpha, beta, old=None):
    """out = RN32(RN32(alpha*linear) + RN32(beta*old)); beta == 0 (either sign)
    never reads `old` (src/transforms.hpp:44-50, docs/API.md:38-45)."""
    value = np.float32(alpha) * np.asarray(linear, dtype=np.float32)
    if float(beta) != 0.0:
        value = value + np.float32(beta) * np.asarray(old, dtype=np.float32)
    return value.astype(np.float32)


def swiglu(gate, up):
    """hidden = RN32(RN32(g*sigmoid(g)) * u) with the stable sigmoid
    e = exp(-|g|) (src/tp_moe_activation.hpp:52-59, tools/make_rank_fixtures.py:170-174)."""
    g = np.asarray(gate, dtype=np.float32)
    u = np.asarray(up, dtype=np.float32)
    e = np.exp(-np.abs(g)).astype(np.float32)
    one = np.float32(1)
    sig = np.where(g < 0, e / (one + e), one / (one + e)).astype(np.float32)
    return ((g * sig).astype(np.float32) * u).astype(np.float32)


def moe_block(x, experts, route_ids, route_scores, alpha=1.0, beta=0.0, old=None, linear=None):
    """Routed-expert block (docs/TP_RANK.md:64-76, src/tp_moe.hip:112-164):
    hidden[r,s] = swiglu(gate_e(x_r), up_e(x_r));
    y_r = alpha * sum_{s ascending, from +0} RN32(score*down_e(hidden)) + beta*old.
    A score of exactly zero skips the slot.  `experts[e]` is a dict with keys
    gate/up/down, each (trellis, suh, svh, k, codebook, bias).  `linear` may be
    supplied to replace the per-projection evaluator (default: staged oracle)."""
    if linear is None:
        def linear(v, w):
            t, su, sv, k, cb, b = w
            return linear_stages(v, t, su, sv, k, cb, b)["output_fp32"]
    x = np.asarray(x, dtype=np.float32)
    ids = np.asarray(route_ids)
    scores = np.asarray(route_scores, dtype=np.float32)
    rows, top_k = ids.shape
    n_out = experts[int(ids[0, 0])]["down"][2].shape[0]
    combined = np.zeros((rows, n_out), dtype=np.float32)
    hidden_all = {}
    for r in range(rows):
        for s in range(top_k):
            if scores[r, s] == 0:
                continue
            e = experts[int(ids[r, s])]
            h = swiglu(linear(x[r:r + 1], e["gate"]), linear(x[r:r + 1], e["up"]))
            hidden_all[(r, s)] = h[0]
            d = linear(h, e["down"])[0]
            combined[r] = combined[r] + scores[r, s] * d
    return apply_alpha_beta(combined, alpha, beta, old), hidden_all


def h128_bounds(total, parts):
    """Split `total` (a multiple of 128) into `parts` contiguous H128-aligned
    ranges, the first `blocks % parts` ranges one block longer.  Generalises the
    two-rank partition of python/strix_trellis/tp.py:78-83 to N ranks."""
    blocks = total // 128
    base, extra = divmod(blocks, parts)
    bounds, begin = [], 0
    for r in range(parts):
        size = base + (1 if r < extra else 0)
        bounds.append((begin * 128, (begin + size) * 128))
        begin += size
    return bounds
