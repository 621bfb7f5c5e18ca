import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

CACHE = os.environ.get("TG_CACHE_DIR", "/tmp")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # keep the file that must run last at the end whatever the collection order
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)


@pytest.fixture(scope="session")
def synth():
    return importlib.import_module("tiny-gemma_b200.synth")


@pytest.fixture(scope="session")
def capi():
    build = importlib.import_module("tiny-gemma_b200.build")
    build.build()
    return importlib.import_module("tiny-gemma_b200.capi")


@pytest.fixture(scope="session")
def port():
    from oracle import build_oracle
    from oracle.oracle_api import Oracle

    build_oracle.build_port()
    return Oracle("port")


@pytest.fixture(scope="session")
def ref():
    """the compiled reference, if oracle/_ref/libtgref.so exists (or can be built here)"""
    from oracle import build_oracle
    from oracle.oracle_api import Oracle, available

    build_oracle.build_ref()
    if not available("reference"):
        pytest.skip("oracle/_ref/libtgref.so not present (reference checkout needed to build it)")
    return Oracle("reference")


@pytest.fixture(scope="session")
def golden():
    g = {}
    for name in ("numpy_modules", "ref_ops", "ref_e2e_270m"):
        g[name] = np.load(os.path.join(ROOT, "tests", "golden", name + ".npz"))
    return g


@pytest.fixture(scope="session")
def weights_270m(synth):
    return synth.write_random_model(os.path.join(CACHE, "tg_270m_s0.bin"), "270m", seed=0)


@pytest.fixture(scope="session")
def weights_1b(synth):
    return synth.write_random_model(os.path.join(CACHE, "tg_1B_s0.bin"), "1B", seed=0)


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def rel_max(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
