"""Shared test plumbing: the `gpu` marker, the package loaded by path, the oracle on sys.path."""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
PKG_DIR = REPO / "llama3-custom-inference_b200"
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def load_package():
    """Imports llama3-custom-inference_b200/ (not a valid identifier) as `llama3_custom_inference_b200`."""
    name = "llama3_custom_inference_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, PKG_DIR / "__init__.py",
                                                  submodule_search_locations=[str(PKG_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def capi(pkg):
    """ctypes view of the C ABI; the library must have been built (build.py / __graft_entry__.build())."""
    pkg.capi.load()
    return pkg.capi


@pytest.fixture(scope="session")
def ext(pkg):
    """The torch extension module `custom_kernels_extension`, imported the way the reference does."""
    return pkg.extension()


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(REPO / "tests" / "golden" / "reference_vectors.pt")


@pytest.fixture(scope="session")
def ref_cuda():
    """Outputs of the reference's own CUDA kernels (tests/golden/make_reference_cuda_golden.py)."""
    import torch

    return torch.load(REPO / "tests" / "golden" / "reference_cuda_vectors.pt")


@pytest.fixture(scope="session")
def device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda", 0)
