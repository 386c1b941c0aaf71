#!/usr/bin/env python3
"""Produce tests/golden/stgpu/ by RUNNING THE REFERENCE's own fixture generator
(tools/make_gpu_fixtures.py in the reference tree, unmodified, synthetic cases only) and
keeping a subset of its 48 STGPU001 files: two per codebook, even and odd rates (odd rates
carry a bias), both orientations.  Each file holds the layer, 32 input rows and every stage
checkpoint computed by the reference's CPU contract.

    python tests/golden/make_stgpu.py --reference <checkout of the reference project>

manifest.json keeps the generator's own records (size, SHA-256, seed) of the kept files.
"""
import argparse
import json
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
KEEP = ("synthetic-mul1-k4-i128-n256", "synthetic-mul1-k5-i256-n128",
        "synthetic-3inst-k2-i256-n128", "synthetic-3inst-k7-i128-n256",
        "synthetic-mcg-k3-i128-n256", "synthetic-mcg-k6-i256-n128")


def main():
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--reference", type=Path, required=True)
    a = p.parse_args()
    out = HERE / "stgpu"
    out.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        subprocess.run([sys.executable, str(a.reference / "tools" / "make_gpu_fixtures.py"), "--out", tmp,
                        "--skip-real"], check=True)
        manifest = json.loads((Path(tmp) / "manifest.json").read_text())
        kept = [r for r in manifest["fixtures"] if Path(r["file"]).stem in KEEP]
        assert len(kept) == len(KEEP)
        for r in kept:
            shutil.copyfile(Path(tmp) / r["file"], out / r["file"])
        manifest.update(fixtures=kept, total_bytes=sum(r["bytes"] for r in kept),
                        note="subset of the generator's 48 synthetic cases")
        (out / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    print(f"kept {len(kept)} files, {manifest['total_bytes']} bytes")


if __name__ == "__main__":
    main()
