import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The C-ABI library must exist before anything imports the package (no fallback path)."""
    from flashinfer_mla_fp4_b200 import build as _b  # noqa: WPS433

    if not _b.LIB_PATH.exists():
        _b.build()
    yield
