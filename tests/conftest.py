"""Shared fixtures. `-m gpu` tests need a B200 and the built CUDA library; everything
else runs on CPU."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    """The package directory is named `mynah-asr_b200` (not an importable identifier);
    it is loaded under the module name `mynah_asr_b200`."""
    if "mynah_asr_b200" in sys.modules:
        return sys.modules["mynah_asr_b200"]
    pkg_dir = os.path.join(ROOT, "mynah-asr_b200")
    spec = importlib.util.spec_from_file_location("mynah_asr_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mynah_asr_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU and the built CUDA library")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def synth():
    load_package()
    import mynah_asr_b200.synth as s
    return s


@pytest.fixture(scope="session")
def gpu_pkg(pkg):
    """The package with the CUDA library loaded; fails (does not skip) when the
    library is missing, so a silent CPU-only pass is impossible."""
    pkg.lib()
    assert pkg.available(), "no sm_100 device: " + pkg.lib().mynah_b200_last_error().decode()
    return pkg
