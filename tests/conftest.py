"""pytest configuration: markers and import path for the in-tree package."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG_DIR = os.path.join(ROOT, "glm-5.2-4x-spark-1x-rtx6k-96gb_b200")


def load_package():
    """Import the in-tree package (its directory name is not a Python identifier)
    under the module name ``glmrt_b200``."""
    if "glmrt_b200" in sys.modules:
        return sys.modules["glmrt_b200"]
    spec = importlib.util.spec_from_file_location(
        "glmrt_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["glmrt_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
