"""Ten million nodes on one GPU (the shape of C4 / C5: 10M x 128, K=32 uint8, M=32): node ids beyond 2^23, 64-bit
offsets into 5 GB of vectors, 320 MB of codes and a 24 GB visited array.  The vectors are a clustered mixture drawn
on the GPU in this run (the oracle checks what the library did with exactly these vectors, so the generator need not
be the benchmark's); the graph is the seeded build (exact kNN graph of the first 65,536 vectors, the others inserted),
which takes seconds where the exact O(n^2) graph takes more than a minute."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF
N, DIM, CLUSTERS = 10_000_000, 128, 1000


@pytest.fixture(scope="module")
def xl(cp):
    import torch
    gen = torch.Generator(device="cuda:0").manual_seed(10)
    centres = torch.randn((CLUSTERS, DIM), generator=gen, device="cuda:0")

    def draw(m):
        out = np.empty((m, DIM), np.float32)
        for i0 in range(0, m, 1 << 20):
            i1 = min(m, i0 + (1 << 20))
            a = torch.randint(0, CLUSTERS, (i1 - i0,), generator=gen, device="cuda:0")
            x = centres[a] + 0.3 * torch.randn((i1 - i0, DIM), generator=gen, device="cuda:0")
            out[i0:i1] = torch.nn.functional.normalize(x, dim=1).cpu().numpy()
        return out

    base, q = draw(N), draw(64)
    del centres
    torch.cuda.empty_cache()
    idx = cp.CPHNSWIndex(DIM, M=32, ef_construction=200, K=32, component_bytes=1)
    idx.set_param("entry_scan", 8192)
    idx.set_param("k_entry", 32)
    idx.set_param("build_seed", 65536)
    idx.add_batch_parallel(base)
    return base, q, idx, idx.codes(), idx.adjacency()


def test_xl_codes_and_knn_rows_beyond_2_pow_23(xl, oracle):
    base, q, idx, codes, adj = xl
    assert idx.size() == N and codes.shape == (N, 32) and adj.shape == (N, 32)
    rows = np.concatenate([np.random.default_rng(1).choice(N, 400, replace=False), np.arange(N - 100, N)])
    signs = oracle.sign_tables(DIM, 32, 42)
    assert np.array_equal(codes[rows], oracle.encode(base[rows], 32, 1, signs, 2))
    assert np.array_equal(idx.get_code(N - 1), codes[N - 1])
    for r0 in (8_400_000, N - 40):  # rows whose ids and whose neighbours' ids exceed 2^23; each against all 10M codes
        want, wd = oracle.knn_graph(codes, 64, r0, r0 + 40)
        got, gd = idx.knn_graph(codes, 64, r0, r0 + 40)
        assert np.array_equal(got, want) and np.array_equal(gd, wd)
        assert np.array_equal(idx.select_neighbors(codes, got, 32, True, r0), oracle.select_neighbors(codes, want, 32, True, r0))


def test_xl_adjacency_and_search(xl, oracle):
    base, q, idx, codes, adj = xl
    valid = adj != INVALID
    assert (adj[valid] < N).all() and valid.sum(axis=1).min() >= 1
    assert not (adj[:: 97] == np.arange(N, dtype=np.uint32)[:: 97, None]).any()
    assert idx.verify_connectivity() > 0.99 * N
    ids, dist, stats = idx.search_and_rerank_batch(q, 10, 100, 500, want_stats=True)
    assert (ids < N).all() and (ids > (1 << 23)).any() and (np.diff(dist, axis=1) >= 0).all()
    exact = -np.einsum("qd,qkd->qk", q, base[ids])
    assert np.allclose(dist, exact, rtol=1e-5, atol=1e-6)
    sample = np.arange(0, q.shape[0], 3)[:20]
    signs = oracle.sign_tables(DIM, 32, 42)
    _, rot, _ = oracle.encode(q[sample], 32, 1, signs, 2, want_rotated=True)
    cand, _, ws = oracle.search(rot, codes, adj, idx.entry_ids(), 500, 500, want_stats=True, n_seed=32)
    wi, wd = oracle.rerank(q[sample], base, cand, 10)
    assert np.array_equal(stats[sample], ws)
    assert np.allclose(dist[sample], wd, rtol=1e-5, atol=1e-6)
    assert (ids[sample] == wi).mean() > 0.99
    pid, pd, ps = idx.search_batch(q[sample], 10, 100, want_stats=True)
    oi, od, os_ = oracle.search(rot, codes, adj, idx.entry_ids(), 100, 10, want_stats=True, n_seed=32)
    assert np.array_equal(pid, oi) and np.array_equal(pd, od) and np.array_equal(ps, os_)
