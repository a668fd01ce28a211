import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The C-ABI library is built in-tree once per session (sources only are committed)."""
    from llcompiler_b200.build import build_all
    build_all()


@pytest.fixture(scope="session", autouse=True)
def _fresh_plan_cache(tmp_path_factory):
    """Every test session gets a plan and weight cache of its own, so that no test depends on what an earlier run left."""
    old = os.environ.get("LLC_CACHE_DIR")
    os.environ["LLC_CACHE_DIR"] = str(tmp_path_factory.mktemp("llc_cache"))
    yield
    if old is None:
        os.environ.pop("LLC_CACHE_DIR", None)
    else:
        os.environ["LLC_CACHE_DIR"] = old
