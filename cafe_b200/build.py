"""Builds libcafe_b200.so in-tree with nvcc for sm_100a.

    python -m cafe_b200.build [--force]

The library is a plain C-ABI shared object (include/cafe_b200.h); nothing here links against torch.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
SO = PKG / "libcafe_b200.so"
SOURCES = ["sketch_cuda.cu", "embed_cuda.cu", "sigmod_cuda.cu", "interact_cuda.cu", "ref_abi.cu", "prof.cu"]
HEADERS = ["cafe_types.h", "cafe_internal.h", "sketch_core.cuh", "sketch_engine.h", "radix_sort.cuh"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]
# the sketch arithmetic must not be contracted into fused multiply-adds: counts are compared bit for bit
PER_FILE = {"sketch_cuda.cu": ["-fmad=false"], "sigmod_cuda.cu": ["-fmad=false"], "ref_abi.cu": ["-fmad=false"], "embed_cuda.cu": [],
            "prof.cu": [], "interact_cuda.cu": []}


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (Path(c).exists() or c == "nvcc"):
            return c
    raise RuntimeError("nvcc not found")


def _stale() -> bool:
    if not SO.exists():
        return True
    t = SO.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [PKG.parent / "include" / "cafe_b200.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return SO
    nvcc = _nvcc()
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    procs = []
    for s in SOURCES:
        obj = objdir / (s + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *PER_FILE[s], "-c", str(CSRC / s), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((s, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for s, obj, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{out}")
        if verbose:
            print(out)
        objs.append(str(obj))
    link = [nvcc, "-shared", "-o", str(SO), *objs, "-lcudart"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
