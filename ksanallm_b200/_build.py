"""In-tree builder for the native parts of the package.

Two shared objects are produced under ``ksanallm_b200/_lib``:

* ``_ksana_host.so``   - pybind11 module with the C++ host runtime (scheduler, KV block manager ...),
  compiled with g++.
* ``libksana_kernels.so`` - every CUDA kernel for sm_100a behind ``extern "C"`` launchers, compiled
  with nvcc (``-gencode arch=compute_100a,code=sm_100a``) and loaded with ctypes.

Sources are rebuilt only when they are newer than the object they produce. The reference drives its
native build through CMake (CMakeLists.txt, cmake/nvidia.cmake:21 lists SM 80-90a); this build
targets sm_100a only and needs no configure step.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "_lib"
OBJ = LIB / "obj"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]


def _newer(src_list, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_list)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build command failed: " + " ".join(str(c) for c in cmd))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)
    return r


def build_host(verbose: bool = False) -> Path:
    import pybind11

    LIB.mkdir(parents=True, exist_ok=True)
    out = LIB / "_ksana_host.so"
    src_dir = CSRC / "host"
    sources = sorted(src_dir.glob("*.cc"))
    deps = sources + sorted(src_dir.glob("*.h"))
    if not _newer(deps, out):
        return out
    cmd = [CXX, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", src_dir,
           *sources, "-o", out, "-lpthread"]
    _run(cmd, verbose)
    return out


def cuda_sources():
    return sorted((CSRC / "cuda").glob("*.cu"))


def build_cuda(verbose: bool = False, ptxas_verbose: bool = False) -> Path:
    LIB.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    out = LIB / "libksana_kernels.so"
    headers = sorted((CSRC / "cuda").glob("*.cuh")) + sorted((CSRC / "cuda").glob("*.h"))
    srcs = cuda_sources()
    if not srcs:
        return out
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if _newer([s, *headers], o):
            cmd = [NVCC, *NVCC_FLAGS, "-I", CSRC / "cuda", "-c", s, "-o", o]
            if ptxas_verbose:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose or ptxas_verbose), jobs))
    if jobs or not out.exists():
        _run([NVCC, "-shared", "-o", out, *objs, "-lcudart"], verbose)
    return out


def build_all(verbose: bool = False) -> None:
    build_host(verbose)
    build_cuda(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built:", *(p.name for p in LIB.glob("*.so")))
