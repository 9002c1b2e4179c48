import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    from oracle.oracle import Port
    return Port()


@pytest.fixture(scope="session")
def ref():
    from oracle.oracle import REF_SO, REFERENCE_ROOT, Ref
    if not REF_SO.exists() and not (REFERENCE_ROOT is not None and (REFERENCE_ROOT / "dabnn" / "bgemm.h").exists()):
        pytest.skip("compiled reference not built and the reference checkout is not present")
    return Ref()
