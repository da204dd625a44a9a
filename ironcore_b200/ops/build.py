"""Build the native sm_100a library in-tree with nvcc.

Every ``csrc/*.cu`` file is compiled with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` into an object file and the
objects are linked into ``ironcore_b200/ops/_native/libironcore_b200.so``. nvcc
cross-compiles without a GPU, so the build runs on a CPU-only machine; the
resulting ``.so`` is loaded through :mod:`ctypes` (plain C ABI, no torch headers,
seconds per file).

Usage: ``python -m ironcore_b200.ops.build [--force] [--verbose]``
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parents[2]
CSRC = REPO_ROOT / "csrc"
OUT_DIR = Path(__file__).resolve().parent / "_native"
LIB_PATH = OUT_DIR / "libironcore_b200.so"
STAMP = OUT_DIR / "build_stamp.json"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-diag-suppress", "177",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    return cand


def _sources():
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not LIB_PATH.exists() or not STAMP.exists():
        return False
    try:
        return json.loads(STAMP.read_text()).get("digest") == _digest()
    except Exception:
        return False


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile all kernels (if sources changed) and return the library path."""
    if not force and is_current():
        return LIB_PATH
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    objs = []

    def compile_one(src: Path):
        obj = OUT_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs),
            "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    STAMP.write_text(json.dumps({"digest": _digest(), "sources": [s.name for s in _sources()]}))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
