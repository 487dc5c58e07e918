import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) and the built libsiglip_fp8.so")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (oracle/libsl8_oracle.so), built on demand where a C compiler exists."""
    from tests.oracle_lib import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def engine():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import siglip_b200
    eng = siglip_b200.Engine(0)
    yield eng
    eng.close()
