"""Seeded synthetic EXL3 layers and activations with the shapes and value
distributions of the benchmark configurations.

Every bit pattern of a trellis tile is a valid code (reference docs/FORMAT.md:58-59),
so uniform random 16-bit containers are a legitimate stand-in for real model
tensors.  Sign/scale vectors are Rademacher signs times |N(0, 0.02)| in float16 and
activations are float16 N(0, 1) widened to float32 for the C ABI, which takes
float32 tensors.  All draws come from numpy.random.Generator(PCG64(seed)).
"""
from dataclasses import dataclass

import numpy as np

BASE_SEED = 20261020  # the reference's fixture base seed (tools/make_gpu_fixtures.py:24)
CODEBOOKS = ("3inst", "mcg", "mul1")


@dataclass
class Layer:
    trellis: np.ndarray      # uint16 [I/16, N/16, 16K]
    suh: np.ndarray          # float16 [I]
    svh: np.ndarray          # float16 [N]
    bias: np.ndarray | None  # float32 [N]
    bits: float  # 1..8, or 1.5 / 2.5 / 3.5 (mul1)
    codebook: str

    @property
    def inputs(self):
        return self.trellis.shape[0] * 16

    @property
    def outputs(self):
        return self.trellis.shape[1] * 16

    @property
    def packed_bytes(self):
        return self.trellis.size * 2


def rng_for(seed):
    return np.random.Generator(np.random.PCG64(seed))


def sign_scale(rng, size, sigma=0.02):
    signs = rng.integers(0, 2, size) * 2 - 1
    return (signs * np.abs(rng.normal(0.0, sigma, size))).astype(np.float16)


def make_layer(inputs, outputs, bits, seed=BASE_SEED, codebook="mul1", bias=False, sigma=0.02):
    if inputs % 128 or outputs % 128:
        raise ValueError("dimensions must be multiples of 128")
    rng = rng_for(seed)
    trellis = rng.integers(0, 65536, (inputs // 16, outputs // 16, int(16 * bits)), dtype=np.uint16)
    suh = sign_scale(rng, inputs, sigma)
    svh = sign_scale(rng, outputs, sigma)
    b = rng.normal(0.0, 0.01, outputs).astype(np.float32) if bias else None
    return Layer(trellis, suh, svh, b, bits, codebook)


def make_activations(rows, inputs, seed=BASE_SEED + 1):
    """float16 N(0,1) rows widened exactly to float32."""
    return rng_for(seed).normal(0.0, 1.0, (rows, inputs)).astype(np.float16).astype(np.float32)


def make_routes(tokens, experts, top_k, seed=BASE_SEED + 2):
    """Router logits ~ N(0,1); the top_k largest per token, softmax over the
    selected logits (the library itself never renormalises scores)."""
    logits = rng_for(seed).normal(0.0, 1.0, (tokens, experts))
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :top_k].astype(np.uint32)
    chosen = np.take_along_axis(logits, ids.astype(np.int64), axis=1)
    e = np.exp(chosen - chosen.max(axis=1, keepdims=True))
    return ids, (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


# ---- the reference's 48-case correctness grid (tools/make_gpu_fixtures.py:62-87) ----
def grid_scales(rng, size):
    values = rng.choice(np.array([-2, -0.5, -0.125, 0, 0.0625, 0.75, 1.5]), size).astype(np.float16)
    values[::17] = 0
    values[1] = np.float16(-0.0)
    return values


def grid_case(codebook_index, bits, wide_input, rows=8):
    """One cell of the grid: bits 1..8 x three codebooks x {(128,256),(256,128)}.
    Returns (layer, x, old, seed).  Row 0 of x holds asymmetric impulses."""
    inputs, outputs = (256, 128) if wide_input else (128, 256)
    seed = BASE_SEED + codebook_index * 1000 + bits * 10 + int(wide_input)
    rng = rng_for(seed)
    trellis = rng.integers(0, 65536, (inputs // 16, outputs // 16, 16 * bits), dtype=np.uint16)
    suh, svh = grid_scales(rng, inputs), grid_scales(rng, outputs)
    bias = rng.normal(0, 0.1, outputs).astype(np.float32) if bits % 2 else None
    layer = Layer(trellis, suh, svh, bias, bits, CODEBOOKS[codebook_index])
    rng2 = rng_for(seed)
    x = rng2.normal(0, 0.25, (rows, inputs)).astype(np.float32)
    x[0] = 0
    x[0, [0, 1, 31, 32, 63, 64, 127, inputs - 1]] = [1, -0.3, 0.7, -1, 0.2, 0.9, -0.4, 0.6]
    old = rng2.normal(0, 0.3, (rows, outputs)).astype(np.float32)
    return layer, x, old, seed
