"""In-tree build of the native parts of aakaar_b200.

Two artefacts, both written next to the sources so that they travel with the tree:

* ``aakaar_b200/lib/libakr_b200.so`` - the CUDA kernels and the C ABI (``include/akr_b200.h``),
  compiled by nvcc for sm_100a only.
* ``aakaar_b200/_C.<abi>.so`` - the pybind11 host module that mirrors the reference's ``_C`` for
  the matmul path and calls the C ABI.

``python -m aakaar_b200._build`` builds both; ``build_all()`` is what ``__graft_entry__.build()`` calls.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libakr_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "static",
]
CUDA_SOURCES = ["gemm_sm100.cu", "aux_kernels.cu", "akr_api.cu", "noalloc.cu", "multi_gpu.cu"]
CUDA_HEADERS = ["gemm_sm100.h", "aux_kernels.h", "sm100_ptx.cuh"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build aakaar_b200")
    return cand


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print("+", " ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build command failed ({res.returncode}): {' '.join(map(str, cmd))}\n{res.stdout}\n{res.stderr}")
    return res


def host_module_path() -> Path:
    return PKG / ("_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    LIBDIR.mkdir(exist_ok=True)
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    headers = [CSRC / h for h in CUDA_HEADERS] + [ROOT / "include" / "akr_b200.h"]
    objs = []
    for src in CUDA_SOURCES:
        obj = objdir / (src + ".o")
        if force or not _newer(obj, [CSRC / src] + headers):
            _run([_nvcc(), *NVCC_FLAGS, "-c", CSRC / src, "-o", obj], verbose)
        objs.append(obj)
    if force or not _newer(LIB, objs):
        _run([_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
              *objs, "-o", LIB, "-Xlinker", "--exclude-libs=ALL", "-lpthread", "-ldl", "-lrt"], verbose)
    return LIB


def build_host(force: bool = False, verbose: bool = False) -> Path:
    import pybind11

    out = host_module_path()
    srcs = [CSRC / "host" / "bindings.cpp"]
    deps = srcs + [CSRC / "host" / "tensor.h", ROOT / "include" / "akr_b200.h", LIB]
    if force or not _newer(out, deps):
        cxx = os.environ.get("CXX", "g++")
        _run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
              f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
              *srcs, "-o", out, f"-L{LIBDIR}", "-lakr_b200", "-Wl,-rpath,$ORIGIN/lib"], verbose)
    return out


def build_microbench(force: bool = False, verbose: bool = False) -> Path:
    """The stand-alone micro-benchmark of the tcgen05.mma instruction stream (csrc/microbench/mma_stream.cu)."""
    LIBDIR.mkdir(exist_ok=True)
    src = CSRC / "microbench" / "mma_stream.cu"
    out = LIBDIR / "mma_stream_bench"
    if force or not _newer(out, [src, CSRC / "sm100_ptx.cuh"]):
        _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-cudart", "static",
              src, "-o", out], verbose)
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_cuda(force, verbose), build_host(force, verbose), build_microbench(force, verbose)


if __name__ == "__main__":
    paths = build_all(force="--force" in sys.argv, verbose=True)
    for p in paths:
        print("built", p)
