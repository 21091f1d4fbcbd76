import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "sparse-winograd-cnn_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import wg_oracle
    wg_oracle.lib()
    return wg_oracle


def pytest_collection_modifyitems(config, items):
    # keep the file order alphabetical so that test_zz_* files run last
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)),))
