import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_small():
    return np.load(GOLDEN / "amo_small.npz")


@pytest.fixture(scope="session")
def golden_extra():
    return np.load(GOLDEN / "codec_extra.npz")


@pytest.fixture(scope="session")
def golden_sym_rows():
    return np.load(GOLDEN / "cache_sym_rows.npz")


@pytest.fixture(scope="session")
def golden_rows():
    return np.load(GOLDEN / "cache_rows.npz")


@pytest.fixture(scope="session")
def digests():
    import json

    return json.loads((GOLDEN / "config_digests.json").read_text())


@pytest.fixture(scope="session")
def built_lib():
    """The C-ABI library, built if needed (nvcc cross-compiles without a GPU)."""
    from tensorcache_b200 import _lib
    from tensorcache_b200 import build as tcb_build

    tcb_build.build()
    return _lib.lib()
