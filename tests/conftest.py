"""Shared test plumbing: import paths, the ``gpu`` marker, library handles."""
import ctypes
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PACKAGE_DIR = ROOT / "consumer-int8-kernels_b200"
for entry in (str(ROOT), str(PACKAGE_DIR)):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ops():
    """The operator module; building it first if the shared objects are not there yet."""
    if not (PACKAGE_DIR / "consumer_int8" / "_C.so").exists():
        subprocess.run([sys.executable, str(PACKAGE_DIR / "build.py")], check=True)
    from consumer_int8 import ops as module

    return module


@pytest.fixture(scope="session")
def c_oracle():
    """The scalar C checker (oracle/ci8_oracle.c), built on demand."""
    target = ROOT / "oracle" / "libci8_oracle.so"
    subprocess.run(["make", "-s", "-C", str(ROOT / "oracle")], check=True)   # rebuilds only when the source is newer
    return ctypes.CDLL(str(target))
