"""The C-ABI library loads and exports every symbol include/cphnsw_b200.h declares; without a GPU
it refuses to work instead of falling back to anything."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cphnsw_b200.h")).read()
    return sorted(set(re.findall(r"\b(cphnsw_b200_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_all_exported(cp):
    lib = cp.load_library()
    names = declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(cp.EXPORTS) == [n for n in names if n in cp.EXPORTS]
    assert set(names) == set(cp.EXPORTS)


def test_no_cpu_fallback(cp):
    """On a machine without a B200 creating an index must fail with a clear CUDA error."""
    if cp.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(cp.CPHNSWError) as e:
        cp.CPHNSWIndex(128)
    assert "no CPU path" in str(e.value) or "CUDA" in str(e.value)


def test_parameter_validation_precedes_device_use(cp):
    # CPHNSWParams::finalize bounds (include/cphnsw/core/types.hpp:403-469) -> std::invalid_argument
    for kwargs in (dict(dim=0), dict(dim=128, K=0), dict(dim=128, K=300), dict(dim=128, M=0), dict(dim=128, M=65),
                   dict(dim=128, M=32, ef_construction=16), dict(dim=128, ef_construction=20000),
                   dict(dim=256, component_bytes=1), dict(dim=128, component_bytes=3), dict(dim=128, fht_convention=9)):
        with pytest.raises(ValueError):
            cp.CPHNSWIndex(**kwargs)


def test_product_never_imports_oracle():
    """Nothing under the package or the library sources may reference the oracle."""
    pkg = os.path.join(ROOT, "sparse-text-kmeans_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.sep + "build" in dirpath:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "liboracle" not in text and "import oracle" not in text and "oracle/" not in text, f
