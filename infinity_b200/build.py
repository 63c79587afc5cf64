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
# The checked build: the same sources with -DB200EMB_BOUNDS=1 (device-side index range checks, csrc/bounds.cuh).
CHECKED_LIB_PATH = LIB_DIR / "libb200emb_checked.so"
CHECKED_OBJ_DIR = PKG_DIR / "build_checked"

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


def _source_digest(extra: str = "") -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    files = sorted(CSRC.glob("*")) + [PKG_DIR.parent / "include" / "b200emb.h"]
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current(checked: bool = False) -> bool:
    stamp = LIB_DIR / ("source_checked.sha256" if checked else "source.sha256")
    lib = CHECKED_LIB_PATH if checked else LIB_PATH
    return lib.exists() and stamp.exists() and stamp.read_text().strip() == _source_digest("checked" if checked else "")


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    """Compile and link the library; returns its path. A no-op when the sources are unchanged.
    ``checked=True`` builds the variant with device-side index range checks beside the normal one."""
    lib_path = CHECKED_LIB_PATH if checked else LIB_PATH
    obj_dir = CHECKED_OBJ_DIR if checked else OBJ_DIR
    if not force and is_current(checked):
        return lib_path
    nvcc = _nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    flags = NVCC_FLAGS + (["-DB200EMB_BOUNDS=1"] if checked else [])

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        (obj_dir / (src.stem + ".ptxas.log")).write_text(proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            print(proc.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(compile_one, sources))
    cmd = [nvcc, "-shared", "-o", str(lib_path), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    if checked:
        (LIB_DIR / "source_checked.sha256").write_text(_source_digest("checked"))
        return lib_path
    (LIB_DIR / "source.sha256").write_text(_source_digest())
    (LIB_DIR / "commit.txt").write_text(source_commit())
    return lib_path


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
    import sys
    print(build(force=True, verbose=True, checked="--checked" in sys.argv[1:]))
