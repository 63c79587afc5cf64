"""Builds the CUDA library in-tree: every ``csrc/*.cu`` is compiled for sm_100a with
nvcc and linked into ``infinity_b200/lib/libb200emb.so`` (no torch, no Python in the
library: it exports the plain C ABI declared in ``include/b200emb.h``).

nvcc cross-compiles without a GPU, so the build also runs on a CPU-only machine.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libb200emb.so"
OBJ_DIR = PKG_DIR / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return exe


def _source_digest() -> str:
    h = hashlib.sha256()
    files = sorted(CSRC.glob("*")) + [PKG_DIR.parent / "include" / "b200emb.h"]
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = LIB_DIR / "source.sha256"
    return LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == _source_digest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the library; returns its path. A no-op when the sources are unchanged."""
    if not force and is_current():
        return LIB_PATH
    nvcc = _nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ_DIR / (src.stem + ".ptxas.log")).write_text(proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            print(proc.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    (LIB_DIR / "source.sha256").write_text(_source_digest())
    (LIB_DIR / "commit.txt").write_text(source_commit())
    return LIB_PATH


def source_commit() -> str:
    """Commit of the checkout the library was built from ("+" appended when files differ from it), or
    "unknown" without git. Written next to the library so that measurement lines can name the build on
    machines that only receive a copy of the tree."""
    try:
        root = str(PKG_DIR.parent)
        head = subprocess.run(["git", "-C", root, "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=10)
        if head.returncode != 0 or not head.stdout.strip():
            return "unknown"
        dirty = subprocess.run(["git", "-C", root, "status", "--porcelain", "--untracked-files=no"], capture_output=True,
                               text=True, timeout=10).stdout.strip()
        return head.stdout.strip() + ("+" if dirty else "")
    except Exception:
        return "unknown"


if __name__ == "__main__":
    print(build(force=True, verbose=True))
