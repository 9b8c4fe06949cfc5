import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_package():
    """Import cheddar-fhe_b200/ (hyphenated directory) as cheddar_fhe_b200."""
    if "cheddar_fhe_b200" in sys.modules:
        return sys.modules["cheddar_fhe_b200"]
    path = os.path.join(ROOT, "cheddar-fhe_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location("cheddar_fhe_b200", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["cheddar_fhe_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def params40(pkg):
    return pkg.load_params("bootparam_40.json")


@pytest.fixture(scope="session")
def oracle40(params40):
    from oracle import Oracle
    return Oracle(params40)


@pytest.fixture(scope="session")
def engine40(pkg, params40):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return pkg.Engine(params40, device=0)
