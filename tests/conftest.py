import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-attention-v100_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


@pytest.fixture(scope="session")
def built_library():
    """Path of the C-ABI library, building it if the sources are newer (nvcc needs no GPU)."""
    sys.path.insert(0, PKG)
    import build as fmha_build  # flash-attention-v100_b200/build.py

    return fmha_build.build_library()
