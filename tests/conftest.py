import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def load_package():
    """Import the hyphen-named package directory as ``mlx_data_b200``."""
    if "mlx_data_b200" in sys.modules:
        return sys.modules["mlx_data_b200"]
    pkg_dir = os.path.join(ROOT, "mlx-data_b200")
    spec = importlib.util.spec_from_file_location(
        "mlx_data_b200", os.path.join(pkg_dir, "__init__.py"), submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mlx_data_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.lib()
    return o


@pytest.fixture(scope="session")
def ctx(pkg):
    c = pkg.Context(device=0, n_lanes=2)
    yield c
    c.close()
