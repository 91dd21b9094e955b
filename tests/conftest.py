import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="session")
def wl(pkg):
    import importlib
    return importlib.import_module("int8_fmha_b200.workloads")


@pytest.fixture(scope="session")
def oracle():
    import __graft_entry__ as ge
    o = ge.load_oracle()
    o.build()
    return o
