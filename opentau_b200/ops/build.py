"""Builds the native libraries in-tree: CUDA sources with nvcc for sm_100a, host-only C++ with g++.

Each ``csrc/<name>.cu`` (and each host source of :data:`HOST_SOURCES`) becomes ``_native/libotb_<name>.so`` (plain
``extern "C"`` entry points, loaded with ctypes — no torch headers, so a full rebuild takes seconds).  Cross-compiles
without a GPU.  Run ``python -m opentau_b200.ops.build`` or call :func:`build_all`.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).parent / "csrc"
OUT = Path(__file__).parent / "_native"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--shared",
              "-Xcompiler", "-fPIC"]
SOURCES = ["gemm_tcgen05", "elementwise", "train_elementwise", "attention_tcgen05", "attention_bwd_tcgen05", "attention_f32", "stss_corr", "comm_p2p", "noalloc_colsum",
           "gemm_dist_tcgen05", "attention_cp_tcgen05", "gemm_skinny_tcgen05"]


#: host-only runtime pieces (no device code): name -> source
HOST_SOURCES = {"bpe": Path(__file__).parent.parent / "runtime" / "csrc" / "bpe.cpp"}
CXX_FLAGS = ["-O3", "-std=c++17", "-shared", "-fPIC", "-pthread"]


def _cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++"):
        if cand and (Path(cand).exists() or shutil.which(cand)):
            return cand
    raise RuntimeError("no C++ compiler found")


def build_host(name: str, force: bool = False) -> Path:
    src = HOST_SOURCES[name]
    OUT.mkdir(exist_ok=True)
    lib, stamp = lib_path(name), OUT / f"{name}.sha256"
    dig = hashlib.sha256(src.read_bytes() + " ".join(CXX_FLAGS).encode()).hexdigest()
    if not force and lib.exists() and stamp.exists() and stamp.read_text() == dig:
        return lib
    res = subprocess.run([_cxx(), *CXX_FLAGS, "-o", str(lib), str(src)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"{_cxx()} failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(dig)
    return lib


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    for f in [src, *sorted(CSRC.glob("*.cuh")), *sorted(CSRC.glob("*.h"))]:
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path(name: str) -> Path:
    return OUT / f"libotb_{name}.so"


def build_one(name: str, force: bool = False, verbose: bool = False) -> Path:
    src = CSRC / f"{name}.cu"
    if not src.exists():
        raise FileNotFoundError(src)
    OUT.mkdir(exist_ok=True)
    lib = lib_path(name)
    stamp = OUT / f"{name}.sha256"
    dig = _digest(src)
    if not force and lib.exists() and stamp.exists() and stamp.read_text() == dig:
        return lib
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(lib), str(src), "-lcudart"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    stamp.write_text(dig)
    return lib


def build_all(force: bool = False, verbose: bool = False) -> list[Path]:
    names = [n for n in SOURCES if (CSRC / f"{n}.cu").exists()]
    with ThreadPoolExecutor(max_workers=min(8, len(names))) as ex:
        built = list(ex.map(lambda n: build_one(n, force, verbose), names))
    return built + [build_host(n, force) for n in HOST_SOURCES]


def main() -> None:
    for p in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print(p)


if __name__ == "__main__":
    main()
