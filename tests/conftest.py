import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def load_package():
    """Import the hyphenated package directory as ``llm_infer_b200``."""
    name = "llm_infer_b200"
    if name in sys.modules:
        return sys.modules[name]
    d = os.path.join(ROOT, "llm-infer_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(d, "__init__.py"),
                                                  submodule_search_locations=[d])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # GPU tests are skipped, not failed, when no device is visible (e.g. `pytest tests` on a CPU box).
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def built_lib(pkg):
    """The product library, compiled if sources changed (nvcc cross-compiles without a GPU)."""
    pkg.build.build_library()
    return pkg.binding.load()


@pytest.fixture(scope="session")
def port():
    import oracle
    if not os.path.exists(oracle.PORT_SO):
        oracle.build()
    return oracle.Oracle("port")


@pytest.fixture(scope="session")
def checker(port):
    """The CPU checker GPU results are compared with: the compiled reference when present, else the port."""
    import oracle
    return oracle.Oracle("reference") if oracle.have_reference() else port
