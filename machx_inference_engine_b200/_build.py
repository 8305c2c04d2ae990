"""In-tree native build: g++ for the host library, nvcc (sm_100a only) for the kernels.

The shared objects land in ``machx_inference_engine_b200/_native/`` so that they travel
with the source tree; nothing is installed into site-packages and nothing is JIT-cached
outside the tree.  ``python -m machx_inference_engine_b200._build`` rebuilds what is stale.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_native"

HOST_LIB = OUT / "libmx_host.so"
CUDA_LIB = OUT / "libmx_cuda.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str | None:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and Path(c).exists():
            return c
    return None


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _stale(lib: Path, srcs: list[Path], extra: str) -> tuple[bool, str]:
    dg = _digest(srcs, extra)
    stamp = lib.with_suffix(".stamp")
    return (not lib.exists() or not stamp.exists() or stamp.read_text() != dg), dg


def _run(cmd: list[str], log: Path | None = None) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("native build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build_host(force: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    hdrs = sorted((CSRC / "host").glob("*.h"))
    OUT.mkdir(exist_ok=True)
    stale, dg = _stale(HOST_LIB, srcs + hdrs, " ".join(GXX_FLAGS))
    if stale or force:
        gxx = shutil.which("g++") or shutil.which("c++")
        if gxx is None:
            raise RuntimeError("no C++ compiler found to build the host library")
        _run([gxx, *GXX_FLAGS, "-shared", *map(str, srcs), "-o", str(HOST_LIB)])
        HOST_LIB.with_suffix(".stamp").write_text(dg)
    return HOST_LIB


def build_cuda(force: bool = False) -> Path:
    srcs = sorted((CSRC / "cuda").glob("*.cu"))
    hdrs = sorted((CSRC / "cuda").glob("*.cuh")) + sorted((CSRC / "cuda").glob("*.h"))
    OUT.mkdir(exist_ok=True)
    stale, dg = _stale(CUDA_LIB, srcs + hdrs, " ".join(NVCC_FLAGS))
    if not (stale or force):
        return CUDA_LIB
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    hdr_dg = _digest(hdrs, " ".join(NVCC_FLAGS))

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        stamp = objdir / (src.stem + ".stamp")
        d = _digest([src], hdr_dg)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != d:
            _run([nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)], log=objdir / (src.stem + ".ptxas.log"))
            stamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *map(str, objs), "-o", str(CUDA_LIB)])
    CUDA_LIB.with_suffix(".stamp").write_text(dg)
    return CUDA_LIB


def build_all(force: bool = False) -> None:
    build_host(force)
    build_cuda(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", HOST_LIB, CUDA_LIB)
