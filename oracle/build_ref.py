"""Compiles the reference's own CUDA extension, unmodified, for sm_100.  TEST INFRASTRUCTURE.

    python oracle/build_ref.py [<reference checkout>]        (default: $L3CI_REFERENCE_CHECKOUT, else DEFAULT_CHECKOUT below)

Sources are compiled where they lie in the checkout (custom_kernels/custom_kernels.cu and
custom_kernels/main.cpp with their two headers); nothing is copied.  The only output is

    oracle/_ref/reference_kernels_sm100.so

a torch extension module with the reference's three functions (custom_kernels/main.cpp:6-8) under a module
name of its own, so that it can never be imported in place of the product's `custom_kernels_extension`.
This takes the place of the reference's setup.py:9-16 (a JIT `torch.utils.cpp_extension.load` with
TORCH_CUDA_ARCH_LIST 8.0-9.0, which yields nothing a B200 can run); the compiler flags are the ones torch's
JIT build passes (`__CUDA_NO_HALF_*` / `__CUDA_NO_BFLOAT16_CONVERSIONS__`, but not
`__CUDA_NO_BFLOAT16_OPERATORS__`, which custom_kernels.cu:365 needs), with the architecture replaced.

What the module is used for:
  * its `rms_norm` and `rot_embed` outputs on seeded inputs pin oracle/rms_norm.py and oracle/rope.py
    (tests/golden/make_reference_cuda_golden.py writes them to a fixture on a GPU box);
  * the three functions are timed beside this repository's kernels as a same-GPU comparator.
Its `flash_attention_decode` is NOT an oracle: the combine kernel indexes every split with blockIdx.z == 0
(custom_kernels/custom_kernels.cu:184,201,209) and does not compute softmax attention beyond 64 tokens.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
MODULE = "reference_kernels_sm100"
OUT = OUT_DIR / (MODULE + ".so")
DEFAULT_CHECKOUT = Path(os.environ.get("L3CI_REFERENCE_CHECKOUT", "/root/reference"))


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(map(str, cmd)), proc.stdout))


def build(checkout: Path = DEFAULT_CHECKOUT, force: bool = False) -> Path:
    """Builds oracle/_ref/reference_kernels_sm100.so from `checkout`; returns its path.  Raises FileNotFoundError
    when the checkout is not there (a GPU box only gets the prebuilt file)."""
    import torch
    from torch.utils import cpp_extension

    src_dir = Path(checkout) / "custom_kernels"
    cu, cpp = src_dir / "custom_kernels.cu", src_dir / "main.cpp"
    deps = [cu, cpp, src_dir / "dtype_bfloat16.cuh", src_dir / "reduce_kernels.cuh", Path(__file__)]
    for d in deps:
        if not d.exists():
            raise FileNotFoundError(d)
    if not force and OUT.exists() and all(d.stat().st_mtime <= OUT.stat().st_mtime for d in deps):
        return OUT
    OUT_DIR.mkdir(exist_ok=True)
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cxx = shutil.which("g++") or "g++"  # the system compiler: see the product's build.py on static libstdc++
    includes = cpp_extension.include_paths(device_type="cuda") + [sysconfig.get_paths()["include"]]
    inc = [a for i in includes for a in ("-isystem", i)]
    common = ["-DTORCH_EXTENSION_NAME=" + MODULE, "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    cu_obj, cpp_obj = OUT_DIR / "custom_kernels.o", OUT_DIR / "main.o"
    _run([nvcc, "-ccbin", cxx, "-gencode", "arch=compute_100,code=sm_100", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
          "--expt-relaxed-constexpr", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
          "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__", *common, *inc,
          "-c", str(cu), "-o", str(cu_obj)])
    _run([cxx, "-O2", "-std=c++17", "-fPIC", *common, *inc, "-c", str(cpp), "-o", str(cpp_obj)])
    torch_lib = Path(torch.__file__).parent / "lib"
    cuda_lib = Path(nvcc).resolve().parent.parent / "lib64"
    _run([cxx, "-shared", str(cu_obj), str(cpp_obj), "-o", str(OUT),
          "-L", str(torch_lib), "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
          "-Wl,-rpath," + str(torch_lib), "-L", str(cuda_lib), "-lcudart"])
    return OUT


def load():
    """Imports the built module (None if it has not been built).  Needs torch imported first."""
    if not OUT.exists():
        return None
    import importlib.util

    import torch  # noqa: F401

    spec = importlib.util.spec_from_file_location(MODULE, OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    path = build(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_CHECKOUT, force="--force" in sys.argv)
    print("built", path, file=sys.stderr)
