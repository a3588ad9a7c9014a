import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "whisper.cpp_b200")


def load_pkg():
    """The package directory name contains a dot, so it is loaded by path under an importable name."""
    if "whisper_cpp_b200" not in sys.modules:
        spec = importlib.util.spec_from_file_location("whisper_cpp_b200", os.path.join(PKG, "__init__.py"),
                                                      submodule_search_locations=[PKG])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["whisper_cpp_b200"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["whisper_cpp_b200"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, ROOT)


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


@pytest.fixture(scope="session")
def model_dir(tmp_path_factory):
    d = os.environ.get("B200_MODEL_DIR") or str(tmp_path_factory.mktemp("models"))
    os.makedirs(d, exist_ok=True)
    return d
