"""In-tree build of the two shared objects of this package, for sm_100a only.

  lib/libl3ci_b200.so                         the kernels behind the C ABI of include/l3ci_b200.h
                                              (nvcc; links the static CUDA runtime, no torch)
  custom_kernels/custom_kernels_extension.so  the torch extension module the reference's model.py
                                              and benchmark_kernel.py import (g++; links torch and
                                              libl3ci_b200.so)

This takes the place of the reference's setup.py:9-16 (a JIT `torch.utils.cpp_extension.load` of
custom_kernels.cu + main.cpp with TORCH_CUDA_ARCH_LIST 8.0-9.0).  It shells out to nvcc / g++
directly so that the artefacts land inside the source tree and nothing depends on a JIT cache.

Run as a script (`python build.py [--force] [--no-extension]`) or call `build_all()`.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OBJ = PKG / "build"
LIB = PKG / "lib" / "libl3ci_b200.so"
EXT = PKG / "custom_kernels" / "custom_kernels_extension.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CUDA_SOURCES = ["host_common.cu", "rms_norm.cu", "rope.cu", "flash_decode.cu", "flash_decode_small.cu", "lse_merge.cu", "greedy_step.cu", "top_p_step.cu", "prefill_attention.cu", "prefill_attention_tc.cu"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put the CUDA toolkit on PATH")


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), proc.stdout))


def _newer(target: Path, deps: list[Path]) -> bool:
    """True if `target` exists and is newer than every dependency."""
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")) + [Path(__file__)]


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles csrc/*.cu into lib/libl3ci_b200.so."""
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    headers = _headers()
    sources = [CSRC / s for s in CUDA_SOURCES if (CSRC / s).exists()]
    jobs = []
    objects = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objects.append(obj)
        if force or not _newer(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        list(pool.map(_run, jobs))
    if force or jobs or not _newer(LIB, objects):
        _run([nvcc, "-shared", "-o", str(LIB), *map(str, objects), "-cudart", "static",
              "-Xlinker", "-soname,libl3ci_b200.so"])
    return LIB


def build_extension(force: bool = False) -> Path:
    """Compiles custom_kernels/main.cpp into the torch extension module."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    src = PKG / "custom_kernels" / "main.cpp"
    if not force and _newer(EXT, [src, LIB] + _headers()):
        return EXT
    # The system g++ on PATH, not $CXX: a toolchain wrapper that links libstdc++ statically puts a second copy
    # of the iostream locale facets into the module, and formatting an integer into an error message
    # then crashes inside a process that already has the shared libstdc++ (torch) loaded.
    cxx = os.environ.get("L3CI_CXX") or shutil.which("g++") or "g++"
    torch_lib = Path(torch.__file__).parent / "lib"
    includes = cpp_extension.include_paths(device_type="cuda")
    includes += [sysconfig.get_paths()["include"], str(INCLUDE)]
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=custom_kernels_extension", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in includes:
        cmd += ["-isystem", inc]
    cmd += [str(src), "-o", str(EXT),
            "-L", str(LIB.parent), "-ll3ci_b200", "-Wl,-rpath,$ORIGIN/../lib",
            "-L", str(torch_lib), "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath," + str(torch_lib)]
    _run(cmd)
    syms = subprocess.run(["nm", "-D", "--defined-only", str(EXT)], stdout=subprocess.PIPE, text=True).stdout
    if "_ZNSt6locale" in syms or "_txnal_" in syms:
        raise RuntimeError(f"{EXT} contains a static copy of libstdc++ (built with {cxx}); use the system g++")
    return EXT


def build_all(force: bool = False, extension: bool = True, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    if extension:
        build_extension(force=force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--force", action="store_true", help="rebuild even if up to date")
    ap.add_argument("--no-extension", action="store_true", help="build only the C-ABI library")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas=-v to nvcc")
    a = ap.parse_args()
    build_all(force=a.force, extension=not a.no_extension, verbose=a.verbose)
    print("built", LIB, "" if a.no_extension else EXT, file=sys.stderr)
