"""Compiles and runs tests/host/test_kdecode3.cpp: the thread-per-row K code-word decode and the V
field unpacking of the tcgen05 decode kernel (byte-permute look-ups, prefix-sum ordinals as gather
selectors, sign handling, words with more than eight outliers, rows with more than 50 outlier
symbols) against plain per-dim decodes, on the CPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_thread_per_row_decode_matches_plain_decode(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no host C++ compiler")
    exe = tmp_path / "test_kdecode3"
    subprocess.run([cxx, "-O2", "-std=c++17", "-I", str(ROOT / "bonsai_mojo_1bit_optimization_t4_cuda_b200" / "csrc"),
                    "-o", str(exe), str(ROOT / "tests" / "host" / "test_kdecode3.cpp")], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.startswith("ok")
