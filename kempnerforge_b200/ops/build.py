"""Builds the native library in-tree with nvcc (sm_100a only).

The kernels are plain CUDA C++ with ``extern "C"`` entry points and no PyTorch
headers, so each translation unit compiles in seconds and the result is one
shared object, ``kempnerforge_b200/lib/libkfb200.so``, loaded through ctypes.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent
REPO_ROOT = PKG_ROOT.parent
CSRC = REPO_ROOT / "csrc"
LIB_DIR = PKG_ROOT / "lib"
LIB_PATH = LIB_DIR / "libkfb200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link them into the shared library (no-op when up to date)."""
    LIB_DIR.mkdir(exist_ok=True)
    stamp = LIB_DIR / "build.stamp"
    fp = _fingerprint()
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text() == fp:
        return LIB_PATH
    nvcc = _nvcc()
    obj_dir = REPO_ROOT / "build" / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    log_dir = REPO_ROOT / "build" / "ptxas"
    log_dir.mkdir(parents=True, exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        (log_dir / (src.stem + ".log")).write_text(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stderr[-4000:]}")
        if verbose:
            print(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(sources())))) as pool:
        objs = list(pool.map(compile_one, sources()))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs),]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
    stamp.write_text(fp)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
