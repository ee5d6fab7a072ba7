"""pytest configuration: marker registration and import paths.

``-m "not gpu"`` runs the oracle against the golden fixtures, the host-side logic and the C-ABI
export check on CPU; ``-m gpu`` runs the parity tests proper on a B200 through the C ABI.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "sparse-text-kmeans_b200"), os.path.join(ROOT, "oracle"), os.path.dirname(__file__)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    import subprocess
    if not os.path.exists(os.path.join(ROOT, "oracle", "liboracle.so")):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")])
    import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def cp():
    """The product package; fails loudly when the CUDA library has not been built."""
    import cphnsw_b200
    cphnsw_b200.load_library()
    return cphnsw_b200
