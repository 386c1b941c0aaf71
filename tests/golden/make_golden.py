#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE's own
Python package (python/strix_trellis in the reference tree).

Run where the reference tree is mounted:
    python tests/golden/make_golden.py --reference <checkout of the reference project>

Inputs are not stored: they are regenerated from seeds by
strix_trellis_b200/synthetic.py, and their SHA-256 is recorded so drift is caught.
What is stored is what the reference computed: SHA-256 of every bit-exact stage
(decoded Q, scaled fp16, input H128, core input, sequential fp32 core, output) and
the float32 outputs themselves for tolerance comparisons.

Files written (STGPU001 containers come from make_stgpu.py):
  grid.json / grid_ref.npz   the reference's 48-case correctness grid (bits 1..8 x
                             3 codebooks x two orientations, 8 rows)
  config1.json / config1.npz 4096x4096 K4 mul1, one fp16 N(0,1) row (benchmark config 1)
  half_rates.json            ring states + decoded Q hashes at rates 1.5/2.5/3.5
  tp_small.npz               H128-aligned output/input slices of a 512x384 K5 layer:
                             per-slice outputs and repacked transport hashes
  moe_small.npz              8 experts, top-3, hidden 256, inter 128, 4 tokens
"""
import argparse
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
from strix_trellis_b200 import synthetic  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "python"))
    import strix_trellis as ref
    from strix_trellis.container import Exl3Tensor

    # ---- 48-case grid -------------------------------------------------------
    cases, outputs = [], {}
    for cb in range(3):
        for bits in range(1, 9):
            for wide in (0, 1):
                layer, x, old, seed = synthetic.grid_case(cb, bits, wide)
                st = ref.matmul_fp32_stages(x, layer.trellis, layer.suh, layer.svh, bits,
                                            layer.codebook, layer.bias)
                name = f"{layer.codebook}-k{bits}-i{layer.inputs}-n{layer.outputs}"
                cases.append(dict(
                    name=name, codebook=cb, bits=bits, wide=wide, seed=seed,
                    inputs_sha=sha(np.concatenate([layer.trellis.ravel().view(np.uint8),
                                                   layer.suh.view(np.uint8), layer.svh.view(np.uint8),
                                                   x.ravel().view(np.uint8), old.ravel().view(np.uint8)])),
                    q=sha(st["rotated_fp16"]), scaled=sha(st["scaled_fp16"]),
                    inh=sha(st["input_hadamard_fp32"]), a=sha(st["core_input_fp16"]),
                    core=sha(st["core_fp32"]), out_h=sha(st["output_hadamard_fp32"]),
                    ref=sha(st["output_fp32"])))
                outputs[name] = st["output_fp32"].astype("<f4")
                outputs[name + ":core"] = st["core_fp32"].astype("<f4")
    (HERE / "grid.json").write_text(json.dumps(dict(rows=8, cases=cases), indent=1) + "\n")
    np.savez_compressed(HERE / "grid_ref.npz", **outputs)

    # ---- config 1 -----------------------------------------------------------
    layer = synthetic.make_layer(4096, 4096, 4, seed=synthetic.BASE_SEED)
    x = synthetic.make_activations(1, 4096)
    q = ref.dequantize_rotated_vectorized(layer.trellis, 4, "mul1")
    assert q[:64].tobytes() == ref.dequantize_rotated(layer.trellis[:4], 4, "mul1").tobytes()
    ins = ref.input_stages_fp32(x, layer.suh)
    core = ref.core_dot_fp32(ins["core_input_fp16"], q)
    outs = ref.output_stages_fp32(core, layer.svh)
    (HERE / "config1.json").write_text(json.dumps(dict(
        inputs=4096, outputs=4096, bits=4, codebook="mul1", seed=synthetic.BASE_SEED,
        x_seed=synthetic.BASE_SEED + 1, trellis_sha=sha(layer.trellis), x_sha=sha(x),
        q=sha(q), a=sha(ins["core_input_fp16"]), core=sha(core), ref=sha(outs["output_fp32"])),
        indent=1) + "\n")
    np.savez_compressed(HERE / "config1.npz", core=core.astype("<f4"),
                        ref=outs["output_fp32"].astype("<f4"))

    # ---- half-integer rates (CPU-only in the reference) -----------------------
    half = {}
    rng = synthetic.rng_for(synthetic.BASE_SEED + 50)
    for rate in (1.5, 2.5, 3.5):
        t = rng.integers(0, 65536, (8, 8, int(16 * rate)), dtype=np.uint16)
        half[str(rate)] = dict(trellis_sha=sha(t), states=sha(ref.unpack_states(t, rate)),
                               q=sha(ref.dequantize_rotated(t, rate, "mul1")))
    (HERE / "half_rates.json").write_text(json.dumps(half, indent=1) + "\n")

    # ---- tensor-parallel slices ----------------------------------------------
    layer = synthetic.make_layer(512, 384, 5, seed=synthetic.BASE_SEED + 60, bias=True)
    x = synthetic.make_activations(3, 512, seed=synthetic.BASE_SEED + 61)
    full = Exl3Tensor(layer.trellis.view(np.int16), layer.suh, layer.svh, 5, "mul1", layer.bias,
                      "synthetic", "w")
    tp = {"full": full.matmul(x, production=True).astype("<f4")}
    for parts in (2, 3):
        for r in range(parts):
            b0, b1 = 128 * (3 * r // parts), 128 * (3 * (r + 1) // parts)
            if b1 > b0:
                part = full.slice_outputs(b0, b1)
                blob, meta = part.transport_blob()
                tp[f"out{parts}_{r}"] = part.matmul(x, production=True).astype("<f4")
                tp[f"out{parts}_{r}_blob_sha"] = np.frombuffer(bytes.fromhex(hashlib.sha256(blob).hexdigest()), np.uint8)
    for parts in (2, 4):
        for r in range(parts):
            a0, a1 = 512 // parts * r, 512 // parts * (r + 1)
            part = full.slice_inputs(a0, a1, include_bias=(r == 0))
            tp[f"in{parts}_{r}"] = part.matmul(x[:, a0:a1], production=True).astype("<f4")
    np.savez_compressed(HERE / "tp_small.npz", **tp)

    # ---- routed experts: every projection is the reference's staged linear ------
    hidden_dim, inter, n_exp, top_k, tokens = 256, 128, 8, 3, 4
    experts = []
    for e in range(n_exp):
        bits = {"gate": 2 + e % 2, "up": 3 if e % 3 == 0 else 2, "down": 2 if e % 3 == 1 else 3}
        experts.append({
            "gate": synthetic.make_layer(hidden_dim, inter, bits["gate"], synthetic.BASE_SEED + 700 + 3 * e, sigma=0.5, bias=True),
            "up": synthetic.make_layer(hidden_dim, inter, bits["up"], synthetic.BASE_SEED + 701 + 3 * e, sigma=0.5),
            "down": synthetic.make_layer(inter, hidden_dim, bits["down"], synthetic.BASE_SEED + 702 + 3 * e, sigma=0.5, bias=True)})
    x = synthetic.make_activations(tokens, hidden_dim, seed=synthetic.BASE_SEED + 790)
    ids, scores = synthetic.make_routes(tokens, n_exp, top_k, seed=synthetic.BASE_SEED + 791)
    scores[1, 2] = 0.0  # a skipped slot

    def lin(v, w):
        return ref.matmul_fp32(v, w.trellis, w.suh, w.svh, w.bits, w.codebook, bias=w.bias)

    hid = np.zeros((tokens, top_k, inter), np.float32)
    each = np.zeros((tokens, top_k, hidden_dim), np.float32)
    y = np.zeros((tokens, hidden_dim), np.float32)
    for r in range(tokens):
        for s in range(top_k):
            if scores[r, s] == 0:
                continue
            e = experts[int(ids[r, s])]
            g, u = lin(x[r:r + 1], e["gate"]), lin(x[r:r + 1], e["up"])
            # the reference's CPU recipe for SwiGLU (tools/make_rank_fixtures.py:169-174)
            ex = np.exp(-np.abs(g)).astype(np.float32)
            sig = np.where(g < 0, ex / (np.float32(1) + ex), np.float32(1) / (np.float32(1) + ex)).astype(np.float32)
            hid[r, s] = ((g * sig).astype(np.float32) * u).astype(np.float32)[0]
            each[r, s] = lin(hid[r, s][None], e["down"])[0]
            y[r] = y[r] + scores[r, s] * each[r, s]
    np.savez_compressed(HERE / "moe_small.npz", ids=ids, scores=scores, hidden=hid, each=each, y=y,
                        x_sha=np.frombuffer(bytes.fromhex(sha(x)), np.uint8))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
