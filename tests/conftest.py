import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def load_package():
    """The package directory carries a hyphen, so it is registered by hand."""
    if "ornith_rs_b200" in sys.modules:
        return sys.modules["ornith_rs_b200"]
    pdir = os.path.join(ROOT, "ornith-rs_b200")
    spec = importlib.util.spec_from_file_location("ornith_rs_b200", os.path.join(pdir, "__init__.py"),
                                                  submodule_search_locations=[pdir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ornith_rs_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def ctx(pkg):
    c = pkg.Context(0)
    yield c
    c.close()
