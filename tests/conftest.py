import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'oracle')):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')


@pytest.fixture(scope='session')
def lib():
    """The built C-ABI library (built here if nvcc is present and it is missing or stale)."""
    from bindcraft2_b200 import _lib, build
    import shutil
    if build.stale() and (shutil.which('nvcc') or os.path.exists('/usr/local/cuda/bin/nvcc')):
        build.build()
    return _lib.load()
