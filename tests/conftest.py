import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def native_lib():
    """The built C-ABI library (compiled on first use)."""
    from tilefusion_b200 import _cabi

    return _cabi.lib()


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np

    data = np.load(ROOT / "tests" / "golden" / "flash_attention_ref.npz")
    meta = json.loads(bytes(data["meta"]).decode())
    return data, meta
