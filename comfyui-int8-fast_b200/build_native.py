"""Builds libi8f.so (the sm_100a CUDA kernels + C ABI) next to this file.

    python comfyui-int8-fast_b200/build_native.py [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library links the static
CUDA runtime, so it only needs the driver at load time.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libi8f.so"
OBJ_DIR = HERE / "build"
SOURCES = ["api.cu", "quant_rowwise.cu", "gemm_tcgen05.cu", "lora_merge_sr.cu", "linear_static.cu",
           "linear_small_m.cu", "peer_barrier.cu", "quant_prologue.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*")) + [HERE.parent / "include" / "i8f.h"]:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = OBJ_DIR / "fingerprint"
    return LIB.exists() and stamp.exists() and stamp.read_text() == _fingerprint()


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and is_current():
        return LIB
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    ptxas = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str) -> Path:
        obj = OBJ_DIR / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *ptxas, "-c", str(CSRC / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            (OBJ_DIR / (Path(src).stem + ".ptxas.log")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    link = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    (OBJ_DIR / "fingerprint").write_text(_fingerprint())
    return LIB


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(out)
