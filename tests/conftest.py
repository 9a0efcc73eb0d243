import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def product():
    """The CUDA product library through its C ABI.  No fallback: a missing library fails."""
    from picoforge_b200 import abi
    api = abi.product()
    assert api.has_extensions
    return api


@pytest.fixture(scope="session")
def gpu(product):
    count = product.lib.qw4cu_device_count()
    assert count > 0, f"no CUDA device: {product.lib.qw4cu_last_error()}"
    assert product.lib.qw4cu_set_device(0) == 0, product.lib.qw4cu_last_error()
    return product
