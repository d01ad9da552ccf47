import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _cuda_ok() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _cuda_ok():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle_c():
    """ctypes handle of the C restatement (built on demand)."""
    import ctypes
    import subprocess

    so = ROOT / "oracle" / "libtuna_oracle.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    lib = ctypes.CDLL(str(so))
    return lib


@pytest.fixture(scope="session")
def tuna_lib():
    from tuna_b200 import _lib, build

    if not _lib.LIB_PATH.exists():
        build.build()
    return _lib.load()
