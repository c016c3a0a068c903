"""pytest configuration: the `gpu` marker, import paths and shared fixtures."""
import ctypes
import importlib
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (hyphenated directory name, hence importlib)."""
    return importlib.import_module("cuda-c-diffusion_b200")


@pytest.fixture(scope="session")
def capi(pkg):
    return importlib.import_module("cuda-c-diffusion_b200.capi")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle binding (test infrastructure)."""
    sys.path.insert(0, str(ROOT / "oracle"))
    mod = importlib.import_module("oracle")
    mod.load()
    mod.set_accumulate_double(True)
    mod.set_threads(1)
    return mod


@pytest.fixture(scope="session")
def lib(capi):
    """Our CUDA library, bound; a missing build is an error, never a skip."""
    return capi.load()


@pytest.fixture(scope="session")
def ref_lib(capi):
    """The reference's own kernels.cu built for sm_100a (oracle/_ref), if present."""
    path = ROOT / "oracle" / "_ref" / "libref_kernels.so"
    if not path.exists():
        pytest.skip("oracle/_ref/libref_kernels.so not built (needs the reference sources at build time)")
    sigs = {k: capi.SIGNATURES[k] for k in capi.REFERENCE_LAUNCHERS}
    return capi.bind(ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL), sigs)


@pytest.fixture(scope="session")
def ref_lib_precise(capi):
    path = ROOT / "oracle" / "_ref" / "libref_kernels_precise.so"
    if not path.exists():
        pytest.skip("oracle/_ref/libref_kernels_precise.so not built")
    sigs = {k: capi.SIGNATURES[k] for k in capi.REFERENCE_LAUNCHERS}
    return capi.bind(ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL), sigs)
