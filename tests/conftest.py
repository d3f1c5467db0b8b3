import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib():
    """The built shared library; builds it first if it is missing."""
    from nnlib_jl_b200 import _lib
    if not _lib.LIB_PATH.exists():
        from nnlib_jl_b200.build import build
        build()
    return _lib.load()


@pytest.fixture(scope="session")
def golden():
    import json
    return json.loads((ROOT / "tests" / "golden" / "nnlib_attention_golden.json").read_text())
