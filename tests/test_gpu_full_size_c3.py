"""The high-dimensional configuration at its full size (C3: 1M x 960 non-negative vectors padded to 1024, uint16
components, K=32, M=32, ef=200, rerank_k=1000): the 1024-point encode kernel, the 11-plane bit-sliced kNN kernel and
the search with the 128 KB query table read in place, each against the oracle on samples of rows and queries (every
stage is per row / per query, so a sample at full size is the full-size computation)."""
import numpy as np
import pytest

from cphnsw_b200 import synthetic

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF


@pytest.fixture(scope="module")
def c3(cp):
    w = synthetic.workload("C3", 1.0)
    w["queries"] = w["queries"][:200]
    idx = cp.CPHNSWIndex(960, M=32, ef_construction=200, K=32, component_bytes=2)
    idx.set_param("entry_scan", w["entry_scan"])
    idx.set_param("k_entry", w.get("k_entry", 4))
    idx.add_batch_parallel(w["base"])
    return w, idx, idx.codes(), idx.adjacency()


def test_c3_full_size_codes_knn_select(c3, oracle):
    w, idx, codes, adj = c3
    n = w["base"].shape[0]
    assert idx.padded_dim == 1024 and codes.dtype == np.uint16 and codes.shape == (n, 32)
    rows = np.random.default_rng(3).choice(n, 500, replace=False)
    signs = oracle.sign_tables(960, 32, 42)
    assert np.array_equal(codes[rows], oracle.encode(w["base"][rows], 32, 2, signs, 2))
    for r0 in (0, 777_777):  # 40 consecutive rows each against all 1M codes, then the pruning
        want, wd = oracle.knn_graph(codes, 64, r0, r0 + 40)
        got, gd = idx.knn_graph(codes, 64, r0, r0 + 40)
        assert np.array_equal(got, want) and np.array_equal(gd, wd)
        sel = idx.select_neighbors(codes, got, 32, True, r0)
        assert np.array_equal(sel, oracle.select_neighbors(codes, want, 32, True, r0))
        assert np.array_equal(sel, adj[r0:r0 + 40])


def test_c3_full_size_search(c3, oracle):
    w, idx, codes, adj = c3
    base, q = w["base"], w["queries"]
    n = base.shape[0]
    k, ef, rr = w["k"], w["ef"], w["rerank_k"]
    out = {}
    for kern in (1, 2):  # one warp and two warps per query, both with the table in global memory
        idx.set_param("search_kernel", kern)
        out[kern] = idx.search_and_rerank_batch(q, k, ef, rr, want_stats=True)
    idx.set_param("search_kernel", 0)
    assert all(np.array_equal(a, b) for a, b in zip(out[1], out[2]))
    ids, dist, stats = out[2]
    assert (ids < n).all() and (np.diff(dist, axis=1) >= 0).all()
    exact = -np.einsum("qd,qkd->qk", q[:50], base[ids[:50]])
    assert np.allclose(dist[:50], exact, rtol=1e-5, atol=1e-6)
    sample = np.arange(0, q.shape[0], 10)  # 20 queries walked by the oracle over the full graph
    signs = oracle.sign_tables(960, 32, 42)
    _, rot, _ = oracle.encode(q[sample], 32, 2, signs, 2, want_rotated=True)
    cand, _, ws = oracle.search(rot, codes, adj, idx.entry_ids(), max(ef, rr, k), rr, want_stats=True, n_seed=w.get("k_entry", 4))
    wi, wd = oracle.rerank(q[sample], base, cand, k)
    assert np.array_equal(stats[sample], ws)
    assert np.allclose(dist[sample], wd, rtol=1e-5, atol=1e-6)
    assert (ids[sample] == wi).mean() > 0.99
    pid, pd, ps = idx.search_batch(q[sample], k, ef, want_stats=True)
    oi, od, os_ = oracle.search(rot, codes, adj, idx.entry_ids(), max(ef, k), k, want_stats=True, n_seed=w.get("k_entry", 4))
    assert np.array_equal(pid, oi) and np.array_equal(pd, od) and np.array_equal(ps, os_)
