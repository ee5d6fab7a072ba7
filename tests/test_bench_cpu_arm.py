"""The CPU arm of bench.py (`--impl reference`) and the tuned build of the oracle it times."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tuned_build_equals_plain_build(oracle):
    """The benchmark's CPU baseline is the oracle's source compiled -O3 -march=native with a sorted-array beam and
    AVX-512 score / byte compare; every result must be the plain checker's."""
    from cphnsw_b200 import synthetic
    base, q = synthetic.gaussian_mixture(6000, 80, 128, 12, 0.3, 77)
    signs = oracle.sign_tables(128, 32, 42)
    codes = oracle.encode(base, 32, 1, signs)
    cand, cd = oracle.knn_graph(codes, 40)
    adj = oracle.select_neighbors(codes, cand, 32, True)
    entry = (np.arange(512, dtype=np.uint64) * 6000 // 512).astype(np.uint32)
    _, rot, _ = oracle.encode(q, 32, 1, signs, want_rotated=True)
    want = [oracle.search(rot, codes, adj, entry, ef, k, want_stats=True, n_seed=ns) for ef, k, ns in ((200, 200, 16), (10, 10, 512), (64, 5, 1))]
    want_sym = oracle.search_codes(codes[:30], codes, adj, entry, 50, 20, n_seed=8)
    want_dist = oracle.code_distance(codes[:50], codes[:400])
    if not oracle.use_tuned_build():
        oracle.use_plain_build()
        import pytest
        pytest.skip("the tuned build does not compile on this host")
    try:
        assert oracle.is_tuned()
        c2, d2 = oracle.knn_graph(codes, 40)
        assert np.array_equal(c2, cand) and np.array_equal(d2, cd)
        assert np.array_equal(oracle.select_neighbors(codes, cand, 32, True), adj)
        got = [oracle.search(rot, codes, adj, entry, ef, k, want_stats=True, n_seed=ns) for ef, k, ns in ((200, 200, 16), (10, 10, 512), (64, 5, 1))]
        for g, w in zip(got, want):
            assert all(np.array_equal(a, b) for a, b in zip(g, w))
        gs = oracle.search_codes(codes[:30], codes, adj, entry, 50, 20, n_seed=8)
        assert all(np.array_equal(a, b) for a, b in zip(gs, want_sym))
        assert np.array_equal(oracle.code_distance(codes[:50], codes[:400]), want_dist)
    finally:
        oracle.use_plain_build()


def test_reference_arm_prints_one_line_with_the_contract_keys():
    env = dict(os.environ, OMP_NUM_THREADS="1")  # what torchrun exports: the arm must not run on one thread because of it
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--scale", "0.02", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "queries/s" and d["higher_is_better"] is True
    assert d["config"]["workload"] == "C2" and d["config"]["cpu_sample"]["index_points"] > 0
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["value"] == d["value"] and d["e2e"]["value"] == d["value"]
    try:
        usable = len(os.sched_getaffinity(0))
    except Exception:
        usable = os.cpu_count()
    assert cb["cores"] == usable
    for key in ("encode", "knn_graph", "select_neighbors", "cpu_model", "nproc", "isa", "ms_per_step"):
        assert key in cb
    assert cb["identical_to_checker"] in (True, None)
    assert 0.5 < d["recall_at_10"] <= 1.0


def test_reference_arm_other_ranks_print_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"], capture_output=True,
                         text=True, timeout=120, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""
