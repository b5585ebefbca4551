import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

entry.load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def _gpu_present() -> bool:
    try:
        import ctypes
        lib = ctypes.CDLL("libcuda.so.1")
        if lib.cuInit(0) != 0:
            return False
        n = ctypes.c_int(0)
        return lib.cuDeviceGetCount(ctypes.byref(n)) == 0 and n.value > 0
    except OSError:
        return False


GPU = _gpu_present()


def pytest_collection_modifyitems(config, items):
    if GPU:
        return
    skip = pytest.mark.skip(reason="no GPU on this machine")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def port(oracle):
    return oracle.Kernels("port")


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"


@pytest.fixture(scope="session")
def tl():
    import importlib
    return importlib.import_module("litespark_inference_b200.torchless")


@pytest.fixture(scope="session")
def kernel(tl):
    import importlib
    return importlib.import_module("litespark_inference_b200.torchless.kernel")


@pytest.fixture(scope="session")
def rng():
    return np.random.default_rng(1234)
