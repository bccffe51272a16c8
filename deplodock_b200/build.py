"""Builds ``libemk.so`` (the C-ABI kernel library) in-tree with nvcc for sm_100a.

The reference compiles generated kernels at run time (``emmy/compiler/backend/cuda/nvcc.py:118-151``: ``nvcc --cubin
-arch=sm_XX[a] --use_fast_math`` with a content-addressed cache). The kernels here are fixed source, so they are
compiled once, ahead of time; nothing is compiled while a program runs. ``--use_fast_math`` is NOT used: the fp32
reductions are held to a 1e-5 relative tolerance against the eager CPU module.

``--bounds-check`` builds the same sources with ``-DEMK_BOUNDS_CHECK`` into ``libemk_check.so``: the variant that
reports out-of-range data-dependent indices (token ids, rotary positions, cu_seqlens) through ``emk_device_status``.
It is loaded instead of ``libemk.so`` when ``EMK_BOUNDS_CHECK=1`` is set (``deplodock_b200.cabi``).

Usage: ``python -m deplodock_b200.build [--force] [--bounds-check]``
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR.parent / "build" / "emk"
LIB_PATH = PKG_DIR / "libemk.so"
CHECK_LIB_PATH = PKG_DIR / "libemk_check.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _source_digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for dep in sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")):
        h.update(dep.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, force: bool, build_dir: Path, flags: list[str]) -> Path:
    obj = build_dir / (src.stem + ".o")
    stamp = build_dir / (src.stem + ".sha")
    digest = _source_digest(src, flags)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj
    cmd = [_nvcc(), *flags, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (build_dir / (src.stem + ".log")).write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(digest)
    return obj


def build(force: bool = False, verbose: bool = False, bounds_check: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libemk.so`` (``bounds_check``: ``libemk_check.so`` with
    ``-DEMK_BOUNDS_CHECK``). Returns the library path."""
    build_dir = BUILD_DIR.parent / "emk_check" if bounds_check else BUILD_DIR
    lib_path = CHECK_LIB_PATH if bounds_check else LIB_PATH
    flags = NVCC_FLAGS + (["-DEMK_BOUNDS_CHECK"] if bounds_check else [])
    build_dir.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, force, build_dir, flags), sources))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if force or not lib_path.exists() or lib_path.stat().st_mtime < newest_obj:
        cmd = [_nvcc(), "-shared", "-o", str(lib_path), *map(str, objs), "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        for s in sources:
            log = (build_dir / (s.stem + ".log")).read_text()
            for line in log.splitlines():
                if "registers" in line or "spill" in line:
                    print(f"[{s.stem}] {line.strip()}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, bounds_check="--bounds-check" in sys.argv)
    print(path)
