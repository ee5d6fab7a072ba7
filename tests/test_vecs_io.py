"""fvecs / ivecs readers and writers (C++ header include/cphnsw/io/vecs_io.hpp and cphnsw_b200/vecs_io.py)
against each other, against committed fixture bytes, and - where the reference checkout was present
when oracle/_ref was built - against the reference's own load_fvecs / load_ivecs / normalize_vectors
(evaluation/datasets/dataset_loader.hpp:40-108,225-240)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from cphnsw_b200 import vecs_io

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
EXE = os.path.join(ROOT, "tests", "cpp", "vecs_io_check")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libcphnsw_ref_scalar.so")


@pytest.fixture(scope="module")
def exe():
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([cxx, "-std=c++17", "-O2", "-ffp-contract=off", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "vecs_io_check.cpp"), "-o", EXE])
    return EXE


def cpp_read(exe, kind, path):
    out = subprocess.run([exe, "read", kind, path], capture_output=True, text=True, check=True).stdout.split()
    dim, count = int(out[0]), int(out[1])
    words = np.array([int(w, 16) for w in out[2:]], np.uint32).reshape(count, dim)
    return words.view(np.float32) if kind == "fvecs" else words


def sample(rng, count, dim):
    x = rng.standard_normal((count, dim)).astype(np.float32)
    if count > 2:
        x[1] = 0.0            # a zero row (normalisation leaves it alone)
        x[2, 0] = np.float32(-0.0)
    return x


@pytest.mark.parametrize("count,dim", [(1, 1), (5, 7), (300, 128), (4097, 3)])
def test_python_and_cpp_agree(tmp_path, exe, count, dim):
    rng = np.random.default_rng(count * 131 + dim)
    x = sample(rng, count, dim)
    ids = rng.integers(0, 2**32, (count, dim), dtype=np.uint64).astype(np.uint32)
    f, i = str(tmp_path / "a.fvecs"), str(tmp_path / "a.ivecs")
    vecs_io.write_fvecs(f, x)
    vecs_io.write_ivecs(i, ids)
    assert os.path.getsize(f) == count * (4 + 4 * dim)
    assert np.array_equal(vecs_io.read_fvecs(f).view(np.uint32), x.view(np.uint32))
    assert np.array_equal(vecs_io.read_ivecs(i), ids)
    assert np.array_equal(cpp_read(exe, "fvecs", f).view(np.uint32), x.view(np.uint32))
    assert np.array_equal(cpp_read(exe, "ivecs", i), ids)
    assert vecs_io.read_fvecs(f, max_count=2).shape == (min(2, count), dim)
    # files written by the C++ writer read back in Python
    g = str(tmp_path / "b.fvecs")
    subprocess.check_call([exe, "write", "fvecs", g, str(count), str(dim)])
    want = (np.arange(count)[:, None] * 1000 + np.arange(dim)[None, :]).astype(np.float32)
    assert np.array_equal(vecs_io.read_fvecs(g), want)


def test_reading_rules(tmp_path, exe):
    """A trailing partial record is ignored; length fields after the first are not checked."""
    x = sample(np.random.default_rng(2), 6, 5)
    f = str(tmp_path / "t.fvecs")
    vecs_io.write_fvecs(f, x)
    raw = bytearray(open(f, "rb").read())
    raw[24:28] = (99).to_bytes(4, "little")  # second record claims another length
    raw += b"\x05\x00\x00\x00\x01\x02"       # partial seventh record
    open(f, "wb").write(raw)
    assert np.array_equal(vecs_io.read_fvecs(f).view(np.uint32), x.view(np.uint32))
    assert np.array_equal(cpp_read(exe, "fvecs", f).view(np.uint32), x.view(np.uint32))
    bad = str(tmp_path / "bad.fvecs")
    open(bad, "wb").write((0).to_bytes(4, "little"))
    with pytest.raises(ValueError):
        vecs_io.read_fvecs(bad)
    assert subprocess.run([exe, "read", "fvecs", bad], capture_output=True).returncode == 2
    assert subprocess.run([exe, "read", "fvecs", str(tmp_path / "missing")], capture_output=True).returncode == 2


def test_committed_fixture(exe):
    """tests/golden/tiny.fvecs / tiny.ivecs were written once by tests/golden/make_golden.py; their
    contents are stored again in vecs_golden.npz."""
    g = np.load(os.path.join(GOLDEN, "vecs_golden.npz"))
    for name, kind in (("tiny.fvecs", "fvecs"), ("tiny.ivecs", "ivecs")):
        path = os.path.join(GOLDEN, name)
        want = g[kind]
        got = vecs_io.read_fvecs(path) if kind == "fvecs" else vecs_io.read_ivecs(path)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert np.array_equal(cpp_read(exe, kind, path).view(np.uint32), want.view(np.uint32))
    assert np.array_equal(vecs_io.normalize_rows(g["fvecs"]).view(np.uint32), g["fvecs_normalized"].view(np.uint32))


def test_normalize_rows_cpp_equals_python(tmp_path, exe):
    x = sample(np.random.default_rng(8), 50, 33) * np.float32(7.5)
    f, g = str(tmp_path / "in.fvecs"), str(tmp_path / "out.fvecs")
    vecs_io.write_fvecs(f, x)
    subprocess.check_call([exe, "norm", f, g])
    got = vecs_io.read_fvecs(g)
    want = vecs_io.normalize_rows(x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.allclose(np.linalg.norm(want[3:], axis=1), 1.0, atol=1e-6) and not want[1].any()


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="reference checkout was not available when oracle/_ref was built")
def test_against_the_reference_loaders(tmp_path):
    ref = C.CDLL(REF_SO)
    if not hasattr(ref, "ref_load_fvecs"):
        pytest.skip("oracle/_ref built without the dataset readers")
    rng = np.random.default_rng(77)
    x = sample(rng, 257, 19) * np.float32(3.0)
    ids = rng.integers(0, 2**31, (40, 100), dtype=np.int64).astype(np.uint32)
    f, i = str(tmp_path / "r.fvecs"), str(tmp_path / "r.ivecs")
    vecs_io.write_fvecs(f, x)
    vecs_io.write_ivecs(i, ids)
    open(f, "ab").write(b"\x13\x00\x00")  # trailing garbage shorter than a record
    dim, count = C.c_uint64(), C.c_uint64()
    out = np.zeros_like(x)
    assert ref.ref_load_fvecs(f.encode(), out.ctypes.data_as(C.c_void_p), C.c_uint64(out.size), C.byref(dim), C.byref(count)) == 0
    assert (dim.value, count.value) == (19, 257)
    assert np.array_equal(out.view(np.uint32), vecs_io.read_fvecs(f).view(np.uint32))
    iout = np.zeros_like(ids)
    assert ref.ref_load_ivecs(i.encode(), iout.ctypes.data_as(C.c_void_p), C.c_uint64(iout.size), C.byref(dim), C.byref(count)) == 0
    assert (dim.value, count.value) == (100, 40)
    assert np.array_equal(iout, vecs_io.read_ivecs(i))
    z = x.copy()
    ref.ref_normalize_vectors(z.ctypes.data_as(C.c_void_p), C.c_uint64(z.shape[0]), C.c_uint64(z.shape[1]))
    assert np.array_equal(z.view(np.uint32), vecs_io.normalize_rows(x).view(np.uint32))
    assert ref.ref_load_fvecs(str(tmp_path / "missing").encode(), None, C.c_uint64(0), C.byref(dim), C.byref(count)) == -1
