import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200); run with -m gpu')


@pytest.fixture(scope='session')
def golden():
    return ROOT / 'tests' / 'golden'


@pytest.fixture(scope='session')
def published(golden):
    import json
    return json.loads((golden / 'reference_published.json').read_text())


@pytest.fixture(scope='session')
def cuda():
    """torch with a CUDA device and the native library loaded; GPU tests fail loudly without either."""
    import torch
    assert torch.cuda.is_available(), 'GPU tests need a CUDA device'
    from deuteron_b200 import native
    native.lib()
    torch.cuda.set_device(0)
    return torch
