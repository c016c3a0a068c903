"""Builds libb200_layer_kernels.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as a script (`python cuda-c-diffusion_b200/build.py [--force]`) or call
`build_library()`.  Objects are compiled in parallel, one nvcc per .cu file, and
linked into `cuda-c-diffusion_b200/libb200_layer_kernels.so`.  nvcc cross-compiles,
so no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libb200_layer_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build libb200_layer_kernels.so")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, force: bool, hdr_mtime: float, extra: list[str]) -> Path:
    obj = BUILD_DIR / (src.stem + ".o")
    if (not force and obj.exists() and obj.stat().st_mtime >= src.stat().st_mtime
            and obj.stat().st_mtime >= hdr_mtime):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return obj


def build_library(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None) -> Path:
    """Compile every csrc/*.cu for sm_100a and link the shared library; returns its path."""
    BUILD_DIR.mkdir(exist_ok=True)
    srcs = sources()
    hdr_mtime = _newest_header_mtime()
    extra = list(extra_flags or [])
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, hdr_mtime, extra), srcs))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest_obj:
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xlinker", "-Bsymbolic", "-o", str(LIB_PATH), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"linked {LIB_PATH}")
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose=True)
    print(path)
