"""Shared fixtures. Tests marked `gpu` need a B200 and call the CUDA library through its C ABI;
everything else runs on CPU (oracle vs the reference build and the golden vectors, host logic,
and that the library loads and exports the whole ABI)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle.bindings import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own ggml build (oracle/_ref); absent where no reference checkout was available."""
    from oracle.bindings import Ref, ref_available
    if not ref_available("base"):
        pytest.skip("oracle/_ref/libtlref_base.so not built (needs a reference checkout: python oracle/build.py)")
    return Ref("base")


@pytest.fixture(scope="session")
def native():
    """One device handle for the whole session; fails loudly if the CUDA library or the GPU is missing."""
    from tensorlisp_b200.native import Native
    n = Native(0)
    yield n
    n.close()
