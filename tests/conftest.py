import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA B200 (sm_100) GPU")


def _have_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def K():
    """The kernels library; built on demand when nvcc is present."""
    from clpeak_b200 import build, native
    if not (native.LIB_DIR / "libclpeak_b200_kernels.so").exists():
        build.build_kernels()
    return native.kernels()


@pytest.fixture(scope="session")
def orc():
    from oracle import binding
    binding.lib()
    return binding


@pytest.fixture(scope="session")
def cuda():
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return torch
