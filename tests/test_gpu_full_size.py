"""The measured configuration at its full size (C2: 1M x 128 clustered, 10k queries, K=32 uint8, M=32,
entry_scan 8192, k_entry 32, ef 100, rerank_k 500): parity with the oracle on samples of rows and
queries (every stage is per row / per query, so a sample at full size is the full-size computation),
and properties that do not depend on the size."""
import numpy as np
import pytest

from cphnsw_b200 import synthetic

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF


@pytest.fixture(scope="module")
def c2(cp):
    w = synthetic.workload("C2", 1.0)
    idx = cp.CPHNSWIndex(128, M=32, ef_construction=200, K=32, component_bytes=1)
    idx.set_param("entry_scan", w["entry_scan"])
    idx.set_param("k_entry", w["k_entry"])
    idx.add_batch_parallel(w["base"])
    return w, idx, idx.codes(), idx.adjacency()


def test_full_size_encode_knn_select_rows(c2, oracle):
    w, idx, codes, adj = c2
    n = w["base"].shape[0]
    rows = np.random.default_rng(0).choice(n, 2000, replace=False)
    signs = oracle.sign_tables(128, 32, 42)
    assert np.array_equal(codes[rows], oracle.encode(w["base"][rows], 32, 1, signs, 2))
    for r0 in (0, 123_456, n - 40):  # 40 consecutive rows each: candidates against all 1M codes, then the pruning
        want, wd = oracle.knn_graph(codes, 64, r0, r0 + 40)
        got, gd = idx.knn_graph(codes, 64, r0, r0 + 40)
        assert np.array_equal(got, want) and np.array_equal(gd, wd)
        sel = idx.select_neighbors(codes, got, 32, True, r0)
        assert np.array_equal(sel, oracle.select_neighbors(codes, want, 32, True, r0))  # the pruning against the oracle's
        assert np.array_equal(sel, adj[r0:r0 + 40])                                    # and the build kept exactly that


def test_full_size_adjacency_properties(c2):
    w, idx, codes, adj = c2
    n = adj.shape[0]
    valid = adj != INVALID
    assert (adj[valid] < n).all()
    assert not (adj == np.arange(n, dtype=np.uint32)[:, None]).any()          # no self loops
    s = np.sort(adj, axis=1)
    assert not ((s[:, 1:] == s[:, :-1]) & (s[:, 1:] != INVALID)).any()         # no id twice in a row
    assert valid.sum(axis=1).min() >= 1
    assert idx.verify_connectivity() > 0.99 * n


def test_full_size_search_parity_and_properties(c2, oracle):
    w, idx, codes, adj = c2
    base, q = w["base"], w["queries"]
    n = base.shape[0]
    k, ef, rr = w["k"], w["ef"], w["rerank_k"]
    out = {}
    for kern in (1, 2):
        idx.set_param("search_kernel", kern)
        out[kern] = idx.search_and_rerank_batch(q, k, ef, rr, want_stats=True)
    idx.set_param("search_kernel", 0)
    ids, dist, stats = out[2]
    assert all(np.array_equal(a, b) for a, b in zip(out[1], out[2]))             # both kernels, all 10k queries
    again = idx.search_and_rerank_batch(q, k, ef, rr, want_stats=True)
    assert all(np.array_equal(a, b) for a, b in zip(again, out[2]))              # idempotent
    assert (ids < n).all() and (np.diff(dist, axis=1) >= 0).all()
    assert all(len(set(r.tolist())) == k for r in ids[:2000])
    assert (stats[:, 0] >= k).all() and (stats[:, 1] >= w["entry_scan"]).all()   # expansions, distance evaluations
    exact = -np.einsum("qd,qkd->qk", q[:500], base[ids[:500]])
    assert np.allclose(dist[:500], exact, rtol=1e-5, atol=1e-6)                  # reranked distances are exact
    # the walk itself against the oracle on a sample of queries over the full graph
    sample = np.arange(0, q.shape[0], 250)
    signs = oracle.sign_tables(128, 32, 42)
    _, rot, _ = oracle.encode(q[sample], 32, 1, signs, 2, want_rotated=True)
    beam = max(ef, rr, k)
    cand, _, ws = oracle.search(rot, codes, adj, idx.entry_ids(), beam, rr, want_stats=True, n_seed=w["k_entry"])
    wi, wd = oracle.rerank(q[sample], base, cand, k)
    assert np.array_equal(stats[sample], ws)
    assert np.allclose(dist[sample], wd, rtol=1e-5, atol=1e-6)
    agree = (ids[sample] == wi).mean()
    assert agree > 0.995  # ids may swap only where two reranked distances tie within the tolerance
    pid, pd, ps = idx.search_batch(q[sample], k, ef, want_stats=True)
    oi, od, os_ = oracle.search(rot, codes, adj, idx.entry_ids(), max(ef, k), k, want_stats=True, n_seed=w["k_entry"])
    assert np.array_equal(pid, oi) and np.array_equal(pd, od) and np.array_equal(ps, os_)


def test_full_size_exact_search(c2, oracle):
    """exact_search over all 1M stored vectors: a sample of queries against the CPU loop (bit-exact), and for
    all 10k queries the size-independent properties (ascending, distinct, distances equal the dot products,
    search_and_rerank never beats the exact k-th distance)."""
    w, idx, codes, adj = c2
    base, q = w["base"], w["queries"]
    ids, dist = idx.exact_search_batch(q, 10)
    assert (ids < base.shape[0]).all() and (np.diff(dist, axis=1) >= 0).all()
    assert all(len(set(r.tolist())) == 10 for r in ids[:2000])
    sample = np.arange(0, q.shape[0], 400)
    wi, wd = oracle.ground_truth(q[sample], base, 10, want_dist=True)
    assert np.array_equal(ids[sample], wi) and np.array_equal(dist[sample], wd)
    exact = -np.einsum("qd,qkd->qk", q[:500], base[ids[:500]])
    assert np.allclose(dist[:500], exact, rtol=1e-5, atol=1e-6)
    ai, ad = idx.search_and_rerank_batch(q, 10, w["ef"], w["rerank_k"])
    assert (ad[:, 9] >= dist[:, 9] - 1e-6).all()          # an approximate top-10 cannot be closer than the exact one
    # rerank of the exact ids gives them back
    ri, rd = idx.rerank_batch(q[:1000], ids[:1000, ::-1].copy(), 10)
    assert np.array_equal(ri, ids[:1000]) and np.array_equal(rd, dist[:1000])
