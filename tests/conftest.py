import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def tables(pkg):
    from saient_quartz_b200.iq_tables import load_tables
    return load_tables()


@pytest.fixture(scope="session")
def oracle_mod(tables):
    import oracle
    oracle.set_tables(tables)
    return oracle


@pytest.fixture(scope="session")
def gpu(pkg):
    """The loaded CUDA library with the IQ codebooks uploaded."""
    pkg.lib()
    pkg.ensure_iq_grids()
    return pkg
