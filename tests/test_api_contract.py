"""Host-side contract of the C ABI without a GPU: the library's own api_*.cpp sources are
compiled with g++ against a counting CUDA runtime (tests/contract/fake/cuda_runtime.h) and
a recording launch layer, and tests/contract/contract_main.cpp asserts the public behaviour
(status precedence, reject-before-allocate, leak-free failure paths, query-free plan submits,
per-device kernel set-up).  Built with the address and undefined-behaviour sanitizers when
the toolchain has them."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CONTRACT = ROOT / "tests" / "contract"
CSRC = ROOT / "strix_trellis_b200" / "csrc"
SOURCES = [CONTRACT / "contract_main.cpp", CONTRACT / "fake_runtime.cpp"] + sorted(CSRC.glob("api_*.cpp"))


def _compile(out, sanitize):
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-Wall", "-Wextra", "-Werror",
           f"-I{CONTRACT / 'fake'}", f"-I{CONTRACT}", f"-I{ROOT / 'include'}", f"-I{CSRC}"]
    if sanitize:
        cmd += ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]
    return subprocess.run(cmd + [str(s) for s in SOURCES] + ["-o", str(out)], capture_output=True, text=True)


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_host_api_contract_against_fake_cuda_runtime(tmp_path):
    exe = tmp_path / "contract"
    built = _compile(exe, sanitize=True)
    if built.returncode:  # a toolchain without the sanitizer runtimes still runs the contract
        built = _compile(exe, sanitize=False)
    assert built.returncode == 0, built.stderr[-4000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "contract ok" in run.stdout
