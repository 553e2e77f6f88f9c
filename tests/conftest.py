import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# every wrapper synchronises and checks the device status word under test
os.environ.setdefault("MCSPARSE_B200_CHECK", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mcsparse_b200 import _lib
    _lib.lib()  # fails loudly if the extension is missing
    return torch.device("cuda", 0)
