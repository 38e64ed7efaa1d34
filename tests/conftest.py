import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_package():
    """Imports the package directory `llama.cu_b200` (not a valid dotted name) as llama_cu_b200."""
    if "llama_cu_b200" in sys.modules:
        return sys.modules["llama_cu_b200"]
    path = os.path.join(ROOT, "llama.cu_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location("llama_cu_b200", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["llama_cu_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU machine)")


@pytest.fixture(scope="session")
def lcu():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle_lib
    oracle_lib.lib()
    return oracle_lib
