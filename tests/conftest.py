import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def reference_root():
    """The leela-zero source tree (present in the build container only)."""
    import oracle as O
    return O.reference_root()


def load_package():
    """Import the package directory ``leela-zero_b200`` (not a valid module
    name, hence by path) as ``leela_zero_b200``."""
    if "leela_zero_b200" in sys.modules:
        return sys.modules["leela_zero_b200"]
    path = os.path.join(ROOT, "leela-zero_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(
        "leela_zero_b200", path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["leela_zero_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def lzb():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.port_lib()
    return O
