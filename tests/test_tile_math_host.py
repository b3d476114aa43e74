"""Builds the host-side test of the tile schedulers' index arithmetic with AddressSanitizer and
UndefinedBehaviorSanitizer and runs it (CPU only; no GPU tool is involved)."""

from __future__ import annotations

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host C++ compiler")
def test_tile_arithmetic_under_sanitizers(tmp_path):
    exe = tmp_path / "test_tile_math"
    flags = ["-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
             "-fno-sanitize-recover=undefined", "-Wall", "-Wextra", "-Werror"]
    build = subprocess.run(["g++", *flags, "-I", str(ROOT / "csrc"), str(ROOT / "tests" / "cpp" / "test_tile_math.cpp"),
                            "-o", str(exe)], capture_output=True, text=True)
    if build.returncode != 0 and ("asan" in build.stderr.lower() or "ubsan" in build.stderr.lower()):
        pytest.skip("sanitizer runtimes are not installed: " + build.stderr.splitlines()[-1])
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "all checks passed" in run.stdout
