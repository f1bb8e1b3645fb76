import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
# The one-GPU emulation of up to eight sequence-parallel ranks runs sixteen streams that wait on
# one another's memory words. With the default of eight hardware queues two streams can share a
# queue, and a waiting stream then holds back the stream that would release it. Must be set
# before the CUDA context exists.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.load_oracle()


@pytest.fixture(scope="session")
def reflib():
    import oracle
    return oracle.load_ref()
