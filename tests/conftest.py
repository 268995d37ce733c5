import importlib.util
import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def load_package():
    """The package directory name is not an identifier; load it by path."""
    name = "adreno_llms_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(REPO, "adreno-llms_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def nnb():
    return load_package()


@pytest.fixture(scope="session")
def built_lib(nnb):
    """Builds the shared library if it is stale (nvcc cross-compiles without a GPU)."""
    spec = importlib.util.spec_from_file_location("nnb_build", os.path.join(REPO, "adreno-llms_b200", "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    b.build()
    return nnb.load()


@pytest.fixture(scope="session")
def ctx(nnb, built_lib):
    c = nnb.Context(0)
    yield c
    c.close()


GOLDEN = os.path.join(REPO, "tests", "golden")
