import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (oracle/librq_oracle.so), built on demand with gcc."""
    from tests import oracle_lib

    return oracle_lib.load()


@pytest.fixture(scope="session")
def rq_ctx():
    """A device context of the product library; GPU tests only."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import recipe_dev_b200 as rq

    ctx = rq.Context(0)
    yield ctx
    ctx.close()
