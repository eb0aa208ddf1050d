"""B200-native decode kernels behind the reference's `custom_kernels_extension` interface.

The directory name is not a Python identifier, so load this package by path, e.g.

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location(
        "llama3_custom_inference_b200", "<repo>/llama3-custom-inference_b200/__init__.py",
        submodule_search_locations=["<repo>/llama3-custom-inference_b200"])
    pkg = importlib.util.module_from_spec(spec); sys.modules[spec.name] = pkg; spec.loader.exec_module(pkg)

Contents:
  build.py        in-tree build of lib/libl3ci_b200.so and custom_kernels/custom_kernels_extension.so
  capi.py         ctypes binding of the C ABI (include/l3ci_b200.h) over torch device tensors
  rope_table.py   rotary table with the Llama-3 frequency scaling as parameters (model.py:27-60)
  sharding.py     partition of a decode batch / a long KV sequence over the GPUs of one box
  decode_loop.py  random-init Llama-3 decode loop around the kernels (end-to-end tokens/s harness)
  custom_kernels/ the torch extension module; put this package directory on sys.path and the
                  reference's `from custom_kernels import custom_kernels_extension` (model.py:23)
                  resolves to it unchanged

There is no CPU or PyTorch fallback anywhere: if a shared object is missing the loaders raise.
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libl3ci_b200.so"
EXT_PATH = PKG_DIR / "custom_kernels" / "custom_kernels_extension.so"


def extension():
    """Imports and returns the torch extension module `custom_kernels_extension`.

    Same import the reference performs (model.py:23, benchmark_kernel.py:4); raises ImportError
    with a build hint if the module has not been built.
    """
    if not EXT_PATH.exists():
        raise ImportError(
            f"{EXT_PATH} is missing: run `python {PKG_DIR / 'build.py'}` (needs nvcc and torch); "
            "there is no fallback implementation")
    if str(PKG_DIR) not in sys.path:
        sys.path.insert(0, str(PKG_DIR))
    import torch  # noqa: F401  (the module links against libtorch)

    return importlib.import_module("custom_kernels.custom_kernels_extension")


from . import capi, decode_loop, rope_table, sharding  # noqa: E402,F401
