"""GPU parity tests: every stage of the CUDA library, called through the C ABI, against the CPU
oracle on the same seeded inputs.  Integer results (codes, code distances, neighbour lists, pruned
lists, graph-walk ids) must be bit-exact; asymmetric distances are bit-exact too (same add order);
reranked distances agree within 1e-5 relative."""
import os

import numpy as np
import pytest

from cphnsw_b200 import synthetic

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "encode_golden.npz"))
CASES = [tuple(int(v) for v in row) for row in GOLD["cases"]]


def make_index(cp, dim, K=32, cb=1, M=32, conv=2, **kw):
    return cp.CPHNSWIndex(dim, M=M, ef_construction=max(200, M), K=K, component_bytes=cb, fht_convention=conv, **kw)


# ---- encode ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("conv", [0, 1, 2])
@pytest.mark.parametrize("ci", range(len(CASES)))
def test_encode_matches_reference_golden(cp, conv, ci):
    dim, K, cb, n = CASES[ci]
    idx = make_index(cp, dim, K, cb, conv=conv)
    P = idx.padded_dim
    bits = np.unpackbits(GOLD["signs_%d" % ci])[: K * 3 * P].reshape(K, 3, P)
    assert np.array_equal(idx.sign_tables(), np.where(bits > 0, 1, -1).astype(np.int8))
    x = GOLD["x_%d" % ci]
    assert np.array_equal(idx.encode(x), GOLD["codes_%d_c%d" % (ci, conv)])
    key = "rot_%d_c%d" % (ci, conv)
    if key in GOLD:
        codes, rot, mag = idx.encode_queries(x[:4])
        assert np.array_equal(codes, GOLD["codes_%d_c%d" % (ci, conv)][:4])
        nz = GOLD[key] != 0
        assert np.array_equal(rot[nz], GOLD[key][nz]) and (rot[~nz] == 0).all()
        assert np.array_equal(mag, GOLD["mag_%d_c%d" % (ci, conv)])


@pytest.mark.parametrize("dim,K,cb,n", [(128, 32, 1, 1), (128, 32, 1, 31), (128, 32, 1, 129), (128, 32, 1, 1000),
                                        (96, 32, 1, 777), (100, 16, 1, 300), (65, 1, 1, 50), (128, 32, 2, 200),
                                        (64, 32, 1, 500), (16, 16, 1, 100), (1, 4, 1, 9), (300, 16, 2, 100),
                                        (960, 32, 2, 70), (1024, 4, 2, 33),
                                        # padded dims 32, 64, 256, 512 (the register / shuffle kernel), 2048 (shared memory)
                                        (20, 8, 1, 333), (33, 16, 1, 257), (256, 32, 2, 300), (200, 32, 2, 129), (512, 8, 2, 65),
                                        (400, 33, 2, 40), (1500, 3, 2, 20)])
@pytest.mark.parametrize("conv", [0, 2])
def test_encode_matches_oracle(cp, oracle, dim, K, cb, n, conv):
    rng = np.random.default_rng(dim * 1000 + n)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    if n > 3:
        x[1] = 0
        x[2] = np.abs(x[2])
    idx = make_index(cp, dim, K, cb, conv=conv)
    signs = oracle.sign_tables(dim, K, 42)
    assert np.array_equal(idx.sign_tables(), signs)
    want, wrot, wmag = oracle.encode(x, K, cb, signs, conv, want_rotated=True)
    assert np.array_equal(idx.encode(x), want)
    codes, rot, mag = idx.encode_queries(x)
    assert np.array_equal(codes, want)
    assert np.array_equal(mag, wmag)
    nz = wrot != 0
    assert np.array_equal(rot[nz], wrot[nz]) and (rot[~nz] == 0).all()


def test_encode_empty_and_custom_signs(cp, oracle):
    idx = make_index(cp, 128)
    assert idx.encode(np.zeros((0, 128), np.float32)).shape == (0, 32)
    rng = np.random.default_rng(5)
    signs = np.where(rng.integers(0, 2, (32, 3, 128)) > 0, 1, -1).astype(np.int8)
    idx.set_sign_tables(signs)
    x = rng.standard_normal((100, 128)).astype(np.float32)
    assert np.array_equal(idx.encode(x), oracle.encode(x, 32, 1, signs, 2))
    with pytest.raises(ValueError):
        idx.set_sign_tables(np.zeros((32, 3, 128), np.int8))


# ---- code distance ---------------------------------------------------------------------------------
@pytest.mark.parametrize("K,cb", [(32, 1), (16, 1), (64, 1), (32, 2), (16, 2), (5, 1), (7, 2), (1, 1), (64, 2), (100, 1), (128, 1), (40, 2)])
def test_code_distance_matches_oracle(cp, oracle, K, cb):
    rng = np.random.default_rng(K * 10 + cb)
    dt = np.uint8 if cb == 1 else np.uint16
    hi = 256 if cb == 1 else 2048
    a = rng.integers(0, hi, (45, K)).astype(dt)
    b = rng.integers(0, hi, (300, K)).astype(dt)
    b[:45] = np.where(rng.random((45, K)) < 0.5, a, b[:45])  # plenty of equal components
    idx = make_index(cp, 128 if cb == 1 else 1024, K, cb)
    assert np.array_equal(idx.code_distance(a, b), oracle.code_distance(a, b))
    assert idx.code_distance(a[:0], b).shape == (0, 300)


# ---- kNN graph ------------------------------------------------------------------------------------------
def clustered_codes(oracle, n, dim, K, cb, seed):
    base, _ = synthetic.gaussian_mixture(n, 1, dim, max(2, n // 200), 0.3, seed)
    return base, oracle.encode(base, K, cb, oracle.sign_tables(dim, K, 42))


@pytest.mark.parametrize("n,k,K,cb,dim", [(1, 4, 32, 1, 128), (2, 4, 32, 1, 128), (33, 40, 32, 1, 128),
                                          (1000, 32, 32, 1, 128), (2500, 64, 32, 1, 128), (3000, 10, 16, 1, 64),
                                          (1500, 32, 32, 2, 256), (1200, 100, 32, 1, 128), (900, 16, 12, 1, 32),
                                          (5000, 32, 32, 1, 96), (2100, 20, 16, 1, 128), (1025, 64, 32, 1, 128),
                                          (1300, 32, 32, 2, 960), (1100, 70, 16, 2, 1000), (2300, 64, 64, 1, 128),
                                          (700, 100, 64, 1, 100), (1400, 64, 64, 2, 300), (1300, 40, 100, 1, 128),
                                          (1030, 20, 128, 1, 64)])  # the last three: 128-byte rows
@pytest.mark.parametrize("kernel", [1, 2])  # byte-wise and bit-sliced distance
def test_knn_graph_matches_oracle(cp, oracle, n, k, K, cb, dim, kernel):
    _, codes = clustered_codes(oracle, n, dim, K, cb, n + k)
    idx = make_index(cp, dim, K, cb)
    sliced_ok = (K in (16, 32, 64) and cb == 1) or (K in (16, 32) and idx.padded_dim == 1024)
    if kernel == 2 and not sliced_ok:
        idx.set_param("knn_kernel", 2)
        with pytest.raises(cp.CPHNSWError):
            idx.knn_graph(codes, k)
        return
    idx.set_param("knn_kernel", kernel)
    nbrs, dist = idx.knn_graph(codes, k)
    wn, wd = oracle.knn_graph(codes, k)
    assert np.array_equal(nbrs, wn)
    assert np.array_equal(dist, wd)
    if n > 64:  # a row block, as a shard would compute it
        rb, re = n // 3, n // 3 + 50
        pn, pd = idx.knn_graph(codes, k, rb, re)
        assert np.array_equal(pn, wn[rb:re]) and np.array_equal(pd, wd[rb:re])


@pytest.mark.parametrize("kernel", [1, 2])
def test_knn_graph_massive_ties_break_by_id(cp, oracle, kernel):
    codes = np.zeros((700, 32), np.uint8)
    codes[::7, 0] = 3  # two classes; within a class every distance is 0
    idx = make_index(cp, 128)
    idx.set_param("knn_kernel", kernel)
    nbrs, dist = idx.knn_graph(codes, 20)
    wn, wd = oracle.knn_graph(codes, 20)
    assert np.array_equal(nbrs, wn) and np.array_equal(dist, wd)


# ---- select_neighbors ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("n,k,M,K,cb,dim,keep", [(1500, 64, 32, 32, 1, 128, True), (1500, 64, 32, 32, 1, 128, False),
                                                 (800, 32, 32, 32, 1, 128, True), (800, 40, 16, 16, 1, 64, True),
                                                 (600, 64, 64, 32, 2, 256, True), (40, 64, 32, 32, 1, 128, True),
                                                 (500, 20, 8, 12, 1, 32, False), (700, 64, 32, 64, 2, 300, True),
                                                 (600, 48, 16, 96, 1, 128, False)])
def test_select_neighbors_matches_oracle(cp, oracle, n, k, M, K, cb, dim, keep):
    _, codes = clustered_codes(oracle, n, dim, K, cb, n + M)
    cand, _ = oracle.knn_graph(codes, k)
    idx = make_index(cp, dim, K, cb, M=M)
    got = idx.select_neighbors(codes, cand, M, keep)
    assert np.array_equal(got, oracle.select_neighbors(codes, cand, M, keep))
    rb = n // 4
    part = idx.select_neighbors(codes, cand[rb:rb + 30], M, keep, row_begin=rb)
    assert np.array_equal(part, got[rb:rb + 30])


# ---- index build + search --------------------------------------------------------------------------------------
def oracle_index(oracle, base, K, cb, M, knn_k, conv=2):
    signs = oracle.sign_tables(base.shape[1], K, 42)
    codes = oracle.encode(base, K, cb, signs, conv)
    cand, _ = oracle.knn_graph(codes, knn_k)
    return signs, codes, oracle.select_neighbors(codes, cand, M, True)


@pytest.mark.parametrize("n,dim,K,cb,M,scan,seeds", [(4000, 128, 32, 1, 32, 64, 4), (4000, 128, 32, 1, 32, 500, 32),
                                                     (3000, 96, 32, 1, 16, 4, 4), (3000, 96, 32, 1, 16, 333, 100),
                                                     (1500, 200, 16, 2, 32, 32, 8), (50, 128, 32, 1, 32, 4, 4),
                                                     (1200, 300, 32, 2, 16, 32, 8), (900, 960, 32, 2, 32, 16, 4),  # table > 32 KB
                                                     (1000, 100, 64, 2, 16, 32, 8),  # 128-byte code rows
                                                     (2000, 128, 64, 1, 32, 64, 8), (1500, 128, 48, 1, 16, 32, 8),  # two rotations per lane in the whole-warp scoring
                                                     (50, 128, 32, 1, 32, 50, 1)])
@pytest.mark.parametrize("skernel", [1, 2])  # one warp per query, two warps per query
def test_build_and_search_match_oracle(cp, oracle, n, dim, K, cb, M, scan, seeds, skernel):
    base, q = synthetic.gaussian_mixture(n, 60, dim, max(2, n // 250), 0.3, n)
    idx = make_index(cp, dim, K, cb, M=M)
    idx.set_param("search_kernel", skernel)
    idx.set_param("entry_scan", scan)
    idx.set_param("k_entry", seeds)
    idx.add_batch_parallel(base)
    assert idx.size() == n
    knn_k = min(64, 2 * M)
    signs, codes, adj = oracle_index(oracle, base, K, cb, M, knn_k)
    assert np.array_equal(idx.codes(), codes)                 # stored code == fresh code
    assert np.array_equal(idx.adjacency(), adj)
    entry = idx.entry_ids()
    assert np.array_equal(entry, (np.arange(min(scan, n), dtype=np.uint64) * n // min(scan, n)).astype(np.uint32))
    _, rot, _ = oracle.encode(q, K, cb, signs, 2, want_rotated=True)
    for k, ef in ((10, 10), (10, 100), (50, 20), (1, 300), (1, 1), (3, 2)):
        ids, dist, stats = idx.search_batch(q, k, ef, want_stats=True)
        wi, wd, ws = oracle.search(rot, codes, adj, entry, max(ef, k), k, want_stats=True, n_seed=seeds)
        assert np.array_equal(ids, wi), (k, ef)
        assert np.array_equal(dist, wd)
        assert np.array_equal(stats, ws)
    # search_and_rerank: the candidate set is bit-exact, reranked distances agree to 1e-5 relative
    for k, ef, rr in ((10, 50, 200), (10, 400, 100), (5, 10, 5)):
        ids, dist = idx.search_and_rerank_batch(q, k, ef, rr)
        cand, _ = oracle.search(rot, codes, adj, entry, max(ef, rr), rr, n_seed=seeds)
        wi, wd = oracle.rerank(q, base, cand, k)
        valid = wi != INVALID
        assert np.array_equal(ids == INVALID, ~valid)
        assert np.allclose(dist[valid], wd[valid], rtol=1e-5, atol=1e-6)
        # ids may differ from the oracle's only where reranked distances tie within the tolerance: an id on
        # one side only must be one of the walk's candidates and lie at the k-th distance
        for qi in range(q.shape[0]):
            if np.array_equal(ids[qi], wi[qi]):
                continue
            kth = float(wd[qi][valid[qi]][-1])
            for node in (set(ids[qi].tolist()) ^ set(wi[qi].tolist())) - {INVALID}:
                assert node in set(cand[qi].tolist()), (qi, node)
                exact = -float(np.dot(q[qi].astype(np.float64), base[node].astype(np.float64)))
                assert abs(exact - kth) <= 1e-5 * abs(kth) + 1e-6, (qi, node, exact, kth)
    # single-query forms return what the batch forms return
    one = idx.search_and_rerank(q[0], 10, 50, 200)
    ids, dist = idx.search_and_rerank_batch(q[:1], 10, 50, 200)
    assert [i for i, _ in one] == [int(i) for i in ids[0] if i != INVALID]


def test_identity_queries_and_ordering(cp):
    # evaluation/qa_protocol.cpp:65-166: querying a stored vector returns its own id first with a
    # negative distance; results ascend
    base, _ = synthetic.gaussian_sphere(3000, 1, 128, 11)
    idx = make_index(cp, 128)
    idx.set_param("entry_scan", 3000)
    idx.add_batch_parallel(base)
    ids, dist = idx.search_and_rerank_batch(base[:50], 10, 100, 200)
    assert (ids[:, 0] == np.arange(50)).all()
    assert np.allclose(dist[:, 0], -1.0, atol=1e-5)
    assert (np.diff(dist, axis=1) >= 0).all()
    ids, dist = idx.search_batch(base[:50], 10, 100)
    assert (ids[:, 0] == np.arange(50)).all() and (dist[:, 0] < 0).all()


def test_add_batch_parallel_appends_and_rebuilds(cp, oracle):
    base, _ = synthetic.gaussian_mixture(1200, 1, 128, 5, 0.3, 9)
    a = make_index(cp, 128)
    a.add_batch(base[:500])            # empty index: the bulk build
    a.add_batch_parallel(base[500:])   # rebuild over everything
    assert a.size() == 1200
    b = make_index(cp, 128)
    b.add_batch_parallel(base)
    assert np.array_equal(a.codes(), b.codes()) and np.array_equal(a.adjacency(), b.adjacency())


def test_seeded_build_is_bulk_seed_plus_insertion(cp):
    """build_seed = s: add_batch_parallel on an empty index builds the exact kNN graph of the first s
    vectors and inserts the others, i.e. exactly add_batch_parallel(x[:s]) followed by add_batch(x[s:])."""
    base, q = synthetic.gaussian_mixture(3000, 20, 128, 12, 0.3, 31)
    a = make_index(cp, 128)
    a.set_param("build_seed", 400)
    a.add_batch_parallel(base)
    b = make_index(cp, 128)
    b.add_batch_parallel(base[:400])
    b.add_batch(base[400:])
    assert a.size() == 3000 and a.get_param("build_seed") == 400
    assert np.array_equal(a.codes(), b.codes()) and np.array_equal(a.adjacency(), b.adjacency())
    c = make_index(cp, 128)
    c.set_param("build_seed", 5000)  # more than there is: the exact graph over everything
    c.add_batch_parallel(base)
    d = make_index(cp, 128)
    d.add_batch_parallel(base)
    assert np.array_equal(c.adjacency(), d.adjacency())
    with pytest.raises(ValueError):
        a.set_param("build_seed", -1)


def oracle_insert(oracle, codes, adj, n_old, m, M, keep, ef_c, entry, n_seed):
    """The declared incremental insertion, step by step with the oracle's pieces: candidates of a new
    node = 64 best of a code-distance walk of the old graph; select_neighbors; every old node chosen
    by new nodes re-selects from (its row + the choosers), the 64 closest by (distance, id)."""
    n = n_old + m
    k_c = min(64, n_old)
    beam = min(1024, max(ef_c, k_c))
    cand, _ = oracle.search_codes(codes[n_old:n], codes[:n_old], adj[:n_old], entry, beam, k_c, n_seed=n_seed)
    full = np.full((n, k_c), INVALID, np.uint32)
    full[n_old:] = cand
    new_rows = oracle.select_neighbors(codes[:n], full, M, keep)[n_old:]
    out = np.concatenate([adj[:n_old], new_rows])
    incoming = {}
    for u in range(n_old, n):
        for v in new_rows[u - n_old]:
            if v < n_old:
                incoming.setdefault(int(v), []).append(u)
    rev = np.full((n, 64), INVALID, np.uint32)
    for v, us in incoming.items():
        ids = [int(w) for w in adj[v] if w != INVALID] + us
        d = oracle.code_distance(codes[v:v + 1], codes[ids])[0]
        order = sorted(zip(d.tolist(), ids))[:64]
        rev[v, :len(order)] = [w for _, w in order]
    sel = oracle.select_neighbors(codes[:n], rev, M, keep)
    for v in incoming:
        out[v] = sel[v]
    return out


@pytest.mark.parametrize("n0,adds,dim,K,cb,M,keep", [(2000, (1, 1, 300, 2500), 128, 32, 1, 32, True), (600, (200,), 300, 64, 2, 16, True),
                                                       (500, (700, 40), 96, 16, 1, 8, False),
                                                       (40, (5, 100), 200, 16, 2, 16, True), (1, (1, 2, 4), 128, 32, 1, 32, True)])
def test_incremental_add_matches_oracle(cp, oracle, n0, adds, dim, K, cb, M, keep):
    total = n0 + sum(adds)
    base, q = synthetic.gaussian_mixture(total, 30, dim, max(2, total // 300), 0.3, total)
    idx = make_index(cp, dim, K, cb, M=M)
    idx.set_param("keep_pruned", int(keep))
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 8)
    idx.add_batch(base[:n0])
    signs = oracle.sign_tables(dim, K, 42)
    codes = oracle.encode(base, K, cb, signs, 2)
    adj = idx.adjacency()
    n = n0
    for a in adds:
        first = idx.add(base[n]) if a == 1 else None
        if a != 1:
            idx.add_batch(base[n:n + a])
        assert first is None or first == n
        # pieces no larger than the graph they join
        done = 0
        while done < a:
            m = min(a - done, n)
            entry = (np.arange(min(64, n), dtype=np.uint64) * n // min(64, n)).astype(np.uint32)
            adj = oracle_insert(oracle, codes, adj, n, m, M, keep, max(200, M), entry, 8)
            n += m
            done += m
        assert idx.size() == n
        assert np.array_equal(idx.codes(), codes[:n])
        assert np.array_equal(idx.adjacency(), adj), (n, a)
    # the grown index searches like any other: ids, distances and counts equal to the oracle's on the same graph
    _, rot, _ = oracle.encode(q, K, cb, signs, 2, want_rotated=True)
    ids, dist, stats = idx.search_batch(q, 5, 40, want_stats=True)
    wi, wd, ws = oracle.search(rot, codes[:n], adj, idx.entry_ids(), 40, 5, want_stats=True, n_seed=8)
    assert np.array_equal(ids, wi) and np.array_equal(dist, wd) and np.array_equal(stats, ws)
    assert idx.verify_connectivity() == oracle.connectivity(adj, idx.entry_ids())


def test_errors_do_not_exit(cp):
    idx = make_index(cp, 128)
    with pytest.raises(cp.CPHNSWError):
        idx.search_batch(np.zeros((1, 128), np.float32), 10, 10)  # empty index
    base, _ = synthetic.gaussian_sphere(100, 1, 128, 1)
    idx.add_batch_parallel(base)
    with pytest.raises(ValueError):
        idx.search_and_rerank_batch(base[:2], 10, 10, 5)  # rerank_k < k
    with pytest.raises(ValueError):
        idx.search_batch(base[:2], 10, 5000)  # beam too wide
    with pytest.raises(ValueError):
        idx.knn_graph(idx.codes(), 500)
    with pytest.raises(ValueError):
        idx.set_param("k_entry", 0)
    ids, _ = idx.search_batch(base[:2], 10, 10)  # still usable
    assert ids.shape == (2, 10)


@pytest.mark.parametrize("skernel", [1, 2])
def test_many_queries_match_oracle(cp, oracle, skernel):
    """Enough queries on a graph large enough that every resident warp (or team of two warps) walks
    many of them concurrently: ids, distances and the per-query expansion/evaluation counts are the
    oracle's, whichever warp scored a neighbour."""
    n, dim, K, M = 20000, 128, 32, 32
    base, q = synthetic.gaussian_mixture(n, 3000, dim, 40, 0.3, 77)
    idx = make_index(cp, dim, K, 1, M=M)
    idx.set_param("search_kernel", skernel)
    idx.set_param("entry_scan", 512)
    idx.set_param("k_entry", 16)
    idx.add_batch_parallel(base)
    codes, adj = idx.codes(), idx.adjacency()
    signs = oracle.sign_tables(dim, K, 42)
    _, rot, _ = oracle.encode(q, K, 1, signs, 2, want_rotated=True)
    for k, ef in ((10, 100), (10, 16)):
        ids, dist, stats = idx.search_batch(q, k, ef, want_stats=True)
        wi, wd, ws = oracle.search(rot, codes, adj, idx.entry_ids(), max(ef, k), k, want_stats=True, n_seed=16)
        assert np.array_equal(ids, wi)
        assert np.array_equal(dist, wd)
        assert np.array_equal(stats, ws)


@pytest.mark.parametrize("skernel", [1, 2])
def test_rows_with_repeated_neighbours_are_offered_once(cp, oracle, skernel):
    """An adjacency installed from outside may list a node twice in a row (the graph builder never
    does): each copy is offered once, as in the sequential walk."""
    import torch
    n, dim, K, M = 5000, 128, 32, 32
    base, q = synthetic.gaussian_mixture(n, 200, dim, 20, 0.3, 13)
    src = make_index(cp, dim, K, 1, M=M)
    src.add_batch_parallel(base)
    codes, adj = src.codes(), src.adjacency().copy()
    rng = np.random.default_rng(3)
    rows = rng.choice(n, n // 2, replace=False)
    adj[rows, 1] = adj[rows, 0]                       # adjacent copies
    adj[rows[: n // 4], 31] = adj[rows[: n // 4], 5]  # distant copies
    adj[rows[: n // 8], 7] = INVALID                  # holes
    idx = make_index(cp, dim, K, 1, M=M)
    idx.set_param("search_kernel", skernel)
    idx.set_param("entry_scan", 256)
    idx.set_param("k_entry", 8)
    dv, dc, da = (torch.from_numpy(x).cuda() for x in (base, codes, adj.view(np.int32)))
    idx.install_dev(dv.data_ptr(), dc.data_ptr(), da.data_ptr(), n)
    signs = oracle.sign_tables(dim, K, 42)
    _, rot, _ = oracle.encode(q, K, 1, signs, 2, want_rotated=True)
    ids, dist, stats = idx.search_batch(q, 10, 200, want_stats=True)
    wi, wd, ws = oracle.search(rot, codes, adj, idx.entry_ids(), 200, 10, want_stats=True, n_seed=8)
    assert np.array_equal(ids, wi) and np.array_equal(dist, wd) and np.array_equal(stats, ws)


@pytest.mark.parametrize("reps", [1, 6000])
def test_two_warp_kernel_wide_beam_on_small_graph(cp, oracle, reps):
    """A beam of 1000 on an unclustered graph of 8000 nodes visits most of it; with many
    repetitions every team of the two-warp kernel passes the wrap of its 8-bit visited epoch
    several times."""
    n, dim, K, M = 8000, 128, 32, 32
    base, q = synthetic.gaussian_sphere(n, 40, dim, 5)
    idx = make_index(cp, dim, K, 1, M=M)
    idx.set_param("search_kernel", 2)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 4)
    idx.add_batch_parallel(base)
    codes, adj = idx.codes(), idx.adjacency()
    signs = oracle.sign_tables(dim, K, 42)
    _, rot, _ = oracle.encode(q, K, 1, signs, 2, want_rotated=True)
    wi, wd, ws = oracle.search(rot, codes, adj, idx.entry_ids(), 1000, 10, want_stats=True, n_seed=4)
    assert ws[:, 1].min() > 5000  # far more marks than any shared-memory set holds
    ids, dist, stats = idx.search_batch(np.tile(q, (reps, 1)), 10, 1000, want_stats=True)
    assert np.array_equal(ids.reshape(reps, 40, 10), np.broadcast_to(wi, (reps, 40, 10)))
    assert np.array_equal(dist.reshape(reps, 40, 10), np.broadcast_to(wd, (reps, 40, 10)))
    assert np.array_equal(stats.reshape(reps, 40, 2), np.broadcast_to(ws, (reps, 40, 2)))


@pytest.mark.parametrize("skernel", [1, 2])
def test_visited_epoch_wraps_without_losing_exactness(cp, oracle, skernel):
    """Each warp stamps visited nodes with an 8-bit per-query epoch; far more than 255 queries per
    warp must keep returning exactly the oracle's answers (the stamp array is zeroed at the wrap)."""
    n, dim, K, M = 1500, 128, 32, 16
    base, q = synthetic.gaussian_mixture(n, 40, dim, 6, 0.3, 321)
    idx = make_index(cp, dim, K, 1, M=M)
    idx.set_param("search_kernel", skernel)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 4)
    idx.add_batch_parallel(base)
    signs, codes, adj = oracle_index(oracle, base, K, 1, M, 32)
    _, rot, _ = oracle.encode(q, K, 1, signs, 2, want_rotated=True)
    wi, wd = oracle.search(rot, codes, adj, idx.entry_ids(), 24, 8, n_seed=4)
    reps = 16000  # 640k queries over at most 148 x 16 warps: every warp passes several wraps
    ids, dist = idx.search_batch(np.tile(q, (reps, 1)), 8, 24)
    assert np.array_equal(ids.reshape(reps, 40, 8), np.broadcast_to(wi, (reps, 40, 8)))
    assert np.array_equal(dist.reshape(reps, 40, 8), np.broadcast_to(wd, (reps, 40, 8)))


# ---- multiprobe ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dim,K,cb,T", [(128, 32, 1, 1), (128, 32, 1, 4), (128, 32, 1, 16), (96, 16, 1, 16), (16, 8, 1, 40),
                                        (200, 16, 2, 16), (128, 3, 1, 64)])
def test_probe_codes_match_oracle(cp, oracle, dim, K, cb, T):
    rng = np.random.default_rng(dim + T)
    q = rng.standard_normal((50, dim)).astype(np.float32)
    q[3] = 0
    q[4, :] = 1.0  # ties everywhere
    idx = make_index(cp, dim, K, cb)
    signs = oracle.sign_tables(dim, K, 42)
    _, rot, _ = oracle.encode(q, K, cb, signs, 2, want_rotated=True)
    assert np.array_equal(idx.probe_codes(q, T), oracle.probe_codes(rot, cb, T))


@pytest.mark.parametrize("n,dim,K,cb,M,T,k,ef", [(3000, 128, 32, 1, 32, 1, 10, 50), (3000, 128, 32, 1, 32, 4, 10, 50),
                                                 (3000, 128, 32, 1, 32, 16, 10, 100), (2000, 96, 16, 1, 16, 16, 5, 20),
                                                 (1500, 200, 16, 2, 32, 4, 10, 40), (1200, 100, 12, 1, 16, 8, 7, 30)])
def test_search_multiprobe_matches_oracle(cp, oracle, n, dim, K, cb, M, T, k, ef):
    base, q = synthetic.gaussian_mixture(n, 40, dim, max(2, n // 250), 0.3, n + T)
    idx = make_index(cp, dim, K, cb, M=M)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 8)
    idx.add_batch_parallel(base)
    signs, codes, adj = oracle_index(oracle, base, K, cb, M, min(64, 2 * M))
    _, rot, _ = oracle.encode(q, K, cb, signs, 2, want_rotated=True)
    wi, wd = oracle.search_multiprobe(rot, cb, codes, adj, idx.entry_ids(), max(ef, k), k, T, n_seed=8)
    ids, dist = idx.search_multiprobe_batch(q, k, ef, T)
    assert np.array_equal(ids, wi)
    assert np.array_equal(dist, wd)
    one = idx.search_multiprobe(q[0], k, ef, T)
    assert [i for i, _ in one] == [int(i) for i in wi[0] if i != INVALID]
    with pytest.raises(ValueError):
        idx.search_multiprobe_batch(q, k, ef, 0)
    with pytest.raises(ValueError):
        idx.search_multiprobe_batch(q, 100, 100, 64)  # num_probes * k too large


# ---- diagnostics around the hot path ---------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("n,dim,K,cb,k", [(3000, 128, 32, 1, 10), (3000, 128, 32, 1, 100), (700, 200, 16, 2, 37),
                                          (50, 128, 32, 1, 64), (2500, 960, 16, 2, 5)])
def test_brute_force_search_matches_oracle(cp, oracle, n, dim, K, cb, k):
    base, q = synthetic.gaussian_mixture(n, 30, dim, max(2, n // 300), 0.3, n + k)
    idx = make_index(cp, dim, K, cb)
    idx.add_batch_parallel(base)
    signs = oracle.sign_tables(dim, K, 42)
    _, rot, _ = oracle.encode(q, K, cb, signs, 2, want_rotated=True)
    ids, dist = idx.brute_force_search_batch(q, k)
    wi, wd = oracle.brute_force(rot, idx.codes(), k)
    assert np.array_equal(ids, wi) and np.array_equal(dist, wd)  # k > n: padded with invalid / +inf on both sides
    assert idx.brute_force_search(q[0], k)[0][0] == int(wi[0, 0])


@pytest.mark.gpu
@pytest.mark.parametrize("n,M,scan", [(4000, 32, 64), (4000, 8, 1), (300, 4, 2), (1, 32, 4)])
def test_verify_connectivity_matches_oracle(cp, oracle, n, M, scan):
    base, _ = synthetic.gaussian_mixture(n, 1, 128, max(2, n // 100), 0.1, 5 * n + M)  # tight clusters: islands at small M
    idx = make_index(cp, 128, M=M)
    idx.set_param("entry_scan", scan)
    idx.set_param("k_entry", 1)
    idx.add_batch_parallel(base)
    want = oracle.connectivity(idx.adjacency(), idx.entry_ids())
    assert idx.verify_connectivity() == want
    assert 1 <= want <= n


@pytest.mark.gpu
@pytest.mark.parametrize("dim,K,cb,m,seed", [(128, 32, 1, 1000, 42), (128, 32, 1, 1, 7), (200, 16, 2, 4096, 1), (64, 8, 1, 333, 99)])
def test_calibrate_matches_oracle(cp, oracle, dim, K, cb, m, seed):
    n = 3000
    base, q = synthetic.gaussian_mixture(n, 50, dim, 10, 0.3, dim + K)
    idx = make_index(cp, dim, K, cb)
    idx.add_batch_parallel(base)
    alpha, beta, r2 = idx.calibrate(m, seed)
    wa, wb, wr, x, y = oracle.calibrate(base, idx.codes(), oracle.sign_tables(dim, K, 42), K, cb, 2, m, seed)
    # samples are bit-exact (same add order on both sides), so the double-precision fits agree to rounding
    assert np.isclose(alpha, wa, rtol=1e-9, atol=1e-12) and np.isclose(beta, wb, rtol=1e-9, atol=1e-12)
    assert np.isclose(r2, wr, rtol=1e-9, atol=1e-12)
    assert idx.get_calibration() == (alpha, beta, r2, m)
    if m >= 333:
        assert alpha > 0 and r2 > 0.2  # the score is positively correlated with the exact distance
    # search_calibrated: ids of search, distances mapped through the fit in fp32
    ids, dist = idx.search_batch(q, 10, 50)
    cids, cdist = idx.search_calibrated_batch(q, 10, 50)
    assert np.array_equal(ids, cids)
    want = np.float32(alpha) * dist + np.float32(beta)
    assert np.array_equal(cdist, want.astype(np.float32))
    # with a rerank the distances are the exact ones
    rids, rdist = idx.search_and_rerank_batch(q, 10, 50, 30)
    crids, crdist = idx.search_calibrated_batch(q, 10, 50, 30)
    assert np.array_equal(rids, crids) and np.array_equal(rdist, crdist)


@pytest.mark.gpu
def test_diagnostics_errors(cp):
    idx = make_index(cp, 128)
    with pytest.raises(cp.CPHNSWError):
        idx.calibrate(100)  # empty index
    assert idx.verify_connectivity() == 0
    base, _ = synthetic.gaussian_sphere(200, 1, 128, 3)
    idx.add_batch_parallel(base)
    with pytest.raises((cp.CPHNSWError, ValueError)):
        idx.calibrate(0)
    with pytest.raises((cp.CPHNSWError, ValueError)):
        idx.brute_force_search_batch(base[:2], 5000)
    assert idx.get_calibration() == (1.0, 0.0, 0.0, 0)


# ---- index file -------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dim,K,cb,M,n", [(128, 32, 1, 32, 3000), (200, 16, 2, 16, 700), (128, 32, 1, 8, 1)])
def test_save_and_load_round_trip(cp, oracle, tmp_path, dim, K, cb, M, n):
    base, q = synthetic.gaussian_mixture(n, 40, dim, max(2, n // 300), 0.3, n + dim)
    a = make_index(cp, dim, K, cb, M=M, seed=7, conv=0)
    a.set_param("entry_scan", 200)
    a.set_param("k_entry", 16)
    a.set_param("keep_pruned", 0)
    a.add_batch_parallel(base)
    if n > 1:
        a.calibrate(500, 3)
    path = str(tmp_path / "index.cphnsw")
    a.save(path)
    assert os.path.getsize(path) == 8 + 104 + K * 3 * a.padded_dim + n * (dim * 4 + K * cb + M * 4)
    b = cp.CPHNSWIndex.load(path)
    assert (b.dim, b.K, b.M, b.component_bytes, b.size()) == (dim, K, M, cb, n)
    assert np.array_equal(a.sign_tables(), b.sign_tables())
    assert np.array_equal(a.codes(), b.codes()) and np.array_equal(a.adjacency(), b.adjacency())
    assert np.array_equal(a.entry_ids(), b.entry_ids())
    assert a.get_calibration() == b.get_calibration()
    assert all(a.get_param(p) == b.get_param(p) for p in ("keep_pruned", "k_entry", "knn_k", "entry_scan", "ef_construction"))
    for k, ef, rr in ((10, 50, 0), (5, 20, 30)):
        k = min(k, n)
        ra = a.search_and_rerank_batch(q, k, ef, max(rr, k)) if rr else a.search_batch(q, k, ef)
        rb = b.search_and_rerank_batch(q, k, ef, max(rr, k)) if rr else b.search_batch(q, k, ef)
        assert np.array_equal(ra[0], rb[0]) and np.array_equal(ra[1], rb[1])
    # a loaded index can be extended like the one that was saved
    extra, _ = synthetic.gaussian_sphere(50, 1, dim, 5)
    a.add_batch_parallel(extra)
    b.add_batch_parallel(extra)
    assert b.size() == n + 50 and np.array_equal(a.adjacency(), b.adjacency())


@pytest.mark.gpu
def test_load_rejects_bad_files(cp, tmp_path):
    idx = make_index(cp, 128)
    base, _ = synthetic.gaussian_sphere(100, 1, 128, 1)
    idx.add_batch_parallel(base)
    path = str(tmp_path / "i.cphnsw")
    idx.save(path)
    raw = open(path, "rb").read()
    # header after the 8-byte magic: 12 32-bit fields, then dim, seed, n as 64-bit fields at bytes 56, 64, 72
    cases = {"magic": b"NOTANIDX" + raw[8:], "version": raw[:8] + (99).to_bytes(4, "little") + raw[12:], "short": raw[:-100],
             "empty": b"", "long": raw + b"\0" * 16,
             "huge_dim": raw[:56] + (1 << 40).to_bytes(8, "little") + raw[64:],
             "huge_n": raw[:72] + (1 << 30).to_bytes(8, "little") + raw[80:],
             "zero_K": raw[:12] + (0).to_bytes(4, "little") + raw[16:]}
    for name, data in cases.items():
        p = str(tmp_path / name)
        open(p, "wb").write(data)
        with pytest.raises(ValueError):
            cp.CPHNSWIndex.load(p)
    with pytest.raises(ValueError):
        cp.CPHNSWIndex.load(str(tmp_path / "missing"))
    with pytest.raises(ValueError):
        idx.save(str(tmp_path / "no_such_dir" / "x"))
    assert idx.search_batch(base[:1], 5, 10)[0].shape == (1, 5)  # still usable


# ---- binary-code mode (the unified index's primary sign-bit code, Hamming metric) -------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("n,dim,K,cb,M", [(3000, 128, 32, 1, 32), (2000, 96, 64, 1, 16), (800, 200, 16, 2, 8), (40, 128, 7, 1, 32)])
def test_binary_mode_matches_oracle(cp, oracle, n, dim, K, cb, M):
    base, q = synthetic.gaussian_mixture(n, 40, dim, max(2, n // 300), 0.3, n + K)
    idx = make_index(cp, dim, K, cb, M=M)
    idx.set_param("binary_codes", 1)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 8)
    idx.add_batch_parallel(base)
    signs = oracle.sign_tables(dim, K, 42)
    codes = (oracle.encode(base, K, cb, signs, 2) & 1).astype(idx.code_dtype)
    qcodes = (oracle.encode(q, K, cb, signs, 2) & 1).astype(idx.code_dtype)
    assert np.array_equal(idx.codes(), codes)            # components are sign bits
    assert np.array_equal(idx.encode(q), qcodes)
    # packed like the unified index's ResidualCode<K,0>::primary.signs
    packed = np.zeros((n, (K + 63) // 64), np.uint64)
    for r in range(K):
        packed[:, r // 64] |= codes[:, r].astype(np.uint64) << np.uint64(r % 64)
    assert np.array_equal(idx.binary_codes(), packed)
    # code distance = Hamming distance; the graph is the oracle's under that distance
    ham = (codes[:50, None, :] != codes[None, :60, :]).sum(axis=2)
    assert np.array_equal(idx.code_distance(codes[:50], codes[:60]), ham)
    knn_k = min(64, 2 * M)
    cand, _ = oracle.knn_graph(codes, knn_k)
    adj = oracle.select_neighbors(codes, cand, M, True)
    assert np.array_equal(idx.adjacency(), adj)
    entry = idx.entry_ids()
    for k, ef in ((10, 50), (5, 5), (1, 200)):
        k = min(k, n)
        ids, dist, stats = idx.search_batch(q, k, ef, want_stats=True)
        wi, wd = oracle.search_codes(qcodes, codes, adj, entry, max(ef, k), k, n_seed=8)
        assert np.array_equal(ids, wi) and np.array_equal(dist, wd)
    # search_and_rerank: Hamming walk, exact rerank of its best rerank_k
    k, ef, rr = min(10, n), 60, min(40, n)
    ids, dist = idx.search_and_rerank_batch(q, k, ef, rr)
    cands, _ = oracle.search_codes(qcodes, codes, adj, entry, max(ef, rr), rr, n_seed=8)
    wi, wd = oracle.rerank(q, base, cands, k)
    valid = wi != INVALID
    assert np.allclose(dist[valid], wd[valid], rtol=1e-5, atol=1e-6) and (ids == wi).mean() > 0.99
    # brute force ranks all nodes by Hamming distance, ties by id
    bi, bd = idx.brute_force_search_batch(q[:10], min(20, n))
    for qi in range(10):
        d = (codes != qcodes[qi]).sum(axis=1)
        order = np.lexsort((np.arange(n), d))[: min(20, n)]
        assert np.array_equal(bi[qi], order.astype(np.uint32)) and np.array_equal(bd[qi], d[order].astype(np.float32))
    # incremental insertion works on sign-bit codes too
    extra, _ = synthetic.gaussian_sphere(30, 1, dim, 8)
    idx.add_batch(extra)
    assert idx.size() == n + 30 and set(np.unique(idx.codes())) <= {0, 1}
    with pytest.raises(cp.CPHNSWError):
        idx.calibrate(100)
    with pytest.raises(cp.CPHNSWError):
        idx.search_multiprobe_batch(q, 5, 10, 4)
    with pytest.raises(cp.CPHNSWError):
        idx.set_param("binary_codes", 0)  # not once vectors have been added


@pytest.mark.gpu
@pytest.mark.parametrize("conv", [0, 1, 2])
@pytest.mark.parametrize("dim", [128, 96, 20])
def test_binary_codes_match_reference_golden(cp, dim, conv):
    """Packed sign codes against the fixture written from the reference's own unified encoder
    (CPEncoder<64,0>, all three FHT builds) and its Hamming kernel (tests/golden/make_binary_golden.py)."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "binary_golden.npz"))
    x = g["x_%d" % dim]
    idx = make_index(cp, dim, 64, 1, conv=conv)
    idx.set_param("binary_codes", 1)
    idx.add_batch_parallel(x)
    assert np.array_equal(idx.binary_codes()[:, 0], g["bits_%d_c%d" % (dim, conv)])
    if dim == 128 and conv == 2:
        codes = idx.codes()
        assert np.array_equal(idx.code_distance(codes[:20], codes), g["hamming_128_c2"].astype(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("K,cb,dim", [(16, 1, 64), (32, 1, 128), (64, 1, 128), (32, 2, 300), (32, 2, 1024), (24, 1, 128),
                                      (96, 1, 128), (120, 1, 64), (8, 1, 32), (20, 1, 128)])
@pytest.mark.parametrize("kernel", [1, 2])
def test_binary_knn_graph_both_kernels(cp, oracle, K, cb, dim, kernel):
    """Sign-bit codes: the bit-sliced kernel runs with one plane per component (K = 16, 32, 64)."""
    n, k = 2200, 48
    _, codes = clustered_codes(oracle, n, dim, K, cb, 7 * K + dim)
    codes = (codes & 1).astype(codes.dtype)
    idx = make_index(cp, dim, K, cb)
    idx.set_param("binary_codes", 1)
    idx.set_param("knn_kernel", kernel)
    if kernel == 2 and K not in (16, 32, 64) and not (cb == 1 and K % 8 == 0):
        with pytest.raises(cp.CPHNSWError):
            idx.knn_graph(codes, k)
        return
    nbrs, dist = idx.knn_graph(codes, k)
    wn, wd = oracle.knn_graph(codes, k)
    assert np.array_equal(nbrs, wn) and np.array_equal(dist, wd)


@pytest.mark.gpu
@pytest.mark.parametrize("dim,K", [(300, 64), (960, 32), (128, 64)])
def test_binary_index_any_dimension(cp, oracle, dim, K):
    """create_binary: one-byte sign components whatever the padded dimension; codes, graph and walk
    equal the oracle's on sign codes."""
    n = 1500
    base, q = synthetic.gaussian_mixture(n, 20, dim, 6, 0.3, dim + K)
    idx = cp.CPHNSWIndex.binary(dim, K=K, M=16)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 8)
    assert idx.get_param("binary_codes") == 1 and idx.get_param("component_bytes") == 1
    idx.add_batch(base)
    signs = oracle.sign_tables(dim, K, 42)
    cb = 1 if idx.padded_dim <= 128 else 2
    codes = (oracle.encode(base, K, cb, signs, 2) & 1).astype(np.uint8)
    qcodes = (oracle.encode(q, K, cb, signs, 2) & 1).astype(np.uint8)
    assert np.array_equal(idx.codes(), codes)
    cand, _ = oracle.knn_graph(codes, 32)
    adj = oracle.select_neighbors(codes, cand, 16, True)
    assert np.array_equal(idx.adjacency(), adj)
    ids, dist = idx.search_batch(q, 10, 80)
    wi, wd = oracle.search_codes(qcodes, codes, adj, idx.entry_ids(), 80, 10, n_seed=8)
    assert np.array_equal(ids, wi) and np.array_equal(dist, wd)



@pytest.mark.gpu
@pytest.mark.parametrize("n,M", [(1200, 16), (20, 32)])
def test_bulk_build_without_pruning_keeps_the_nearest(cp, oracle, n, M):
    """prune = 0 (build_with_gpu_knn(..., prune = false)): the links are the M nearest by (code distance, id)."""
    base, q = synthetic.gaussian_mixture(n, 10, 64, 5, 0.3, 77)
    idx = cp.CPHNSWIndex(64, K=16, M=M)
    idx.set_param("prune", 0)
    assert idx.get_param("prune") == 0
    idx.add_batch_parallel(base)
    codes = oracle.encode(base, 16, 1, oracle.sign_tables(64, 16, 42), 2)
    cand, _ = oracle.knn_graph(codes, M)
    assert np.array_equal(idx.adjacency(), cand)
    _, rot, _ = idx.encode_queries(q)
    ids, dist = idx.search_batch(q, 5, 40)
    wi, wd = oracle.search(rot, codes, cand, idx.entry_ids(), 40, 5, n_seed=min(4, n))
    assert np.array_equal(ids, wi) and np.array_equal(dist, wd)


@pytest.mark.gpu
@pytest.mark.parametrize("n,nq,dim,k", [(5000, 70, 128, 10), (3000, 33, 100, 40), (2600, 9, 960, 100), (700, 300, 17, 128),
                                        (5, 3, 64, 10), (40000, 1000, 64, 1)])
def test_exact_search_equals_cpu_ground_truth(cp, oracle, n, nq, dim, k):
    """exact_search (GPUBruteForce::search, the harness's ground truth): ids and distances of the k smallest
    (-<q,x>, id), bit for bit, for every k class, a dimension that is not a multiple of 4, a split base and
    an index smaller than k."""
    base, q = synthetic.gaussian_mixture(n, nq, dim, max(1, n // 200), 0.3, 5 + dim)
    base[1] = base[0]  # equal distances: ties go to the lower id
    idx = cp.CPHNSWIndex(dim, K=16, M=8, component_bytes=1 if dim <= 128 else 2)
    idx.set_exact_base(base)
    ids, dist = idx.exact_search_batch(q, k)
    wi, wd = oracle.ground_truth(q, base, k, want_dist=True)
    assert np.array_equal(ids, wi)
    assert np.array_equal(dist, wd)
    # queries equal to base rows: the row itself comes first with distance -|x|^2
    ids2, _ = idx.exact_search_batch(base[:4], 1)
    assert list(ids2[:, 0]) == [0, 0, 2, 3]
    idx.set_exact_base(None)
    with pytest.raises(cp.CPHNSWError):
        idx.exact_search_batch(q, k)  # no vectors left


@pytest.mark.gpu
def test_exact_search_runs_over_the_index_vectors_by_default(cp, oracle):
    base, q = synthetic.gaussian_mixture(3000, 50, 128, 10, 0.3, 9)
    idx = cp.CPHNSWIndex(128, K=16, M=16)
    idx.add_batch_parallel(base)
    ids, dist = idx.exact_search_batch(q, 10)
    wi, wd = oracle.ground_truth(q, base, 10, want_dist=True)
    assert np.array_equal(ids, wi) and np.array_equal(dist, wd)
    with pytest.raises(ValueError):
        idx.exact_search_batch(q, 129)


@pytest.mark.gpu
@pytest.mark.parametrize("dim,k,ncand", [(128, 10, 200), (100, 5, 33), (64, 100, 150), (64, 20, 7)])
def test_rerank_batch_equals_cpu(cp, oracle, dim, k, ncand):
    """rerank (GPUBruteForce::rerank): candidates in any order, with holes and repeats."""
    n, nq = 4000, 37
    base, q = synthetic.gaussian_mixture(n, nq, dim, 20, 0.3, 3 + k)
    rng = np.random.default_rng(k)
    cand = rng.integers(0, n, size=(nq, ncand)).astype(np.uint32)
    cand[:, ::7] = 0xFFFFFFFF
    cand[:, 1] = cand[:, 2]
    idx = cp.CPHNSWIndex(dim, K=16, M=8)
    idx.set_exact_base(base)
    ids, dist = idx.rerank_batch(q, cand, k)
    wi, wd = oracle.rerank(q, base, cand, k)
    assert np.array_equal(ids, wi)
    assert np.array_equal(dist, wd)


def residual_index(cp, dim, Kp, R, shift, M=16, conv=2):
    idx = cp.CPHNSWIndex.binary(dim, K=Kp + R, M=M, fht_convention=conv)
    idx.set_param("residual_bits", R)
    idx.set_param("residual_shift", shift)
    return idx


@pytest.mark.gpu
@pytest.mark.parametrize("conv", [0, 1, 2])
@pytest.mark.parametrize("dim", [128, 100, 24])
def test_residual_codes_match_reference_golden(cp, dim, conv):
    """Codes against the reference's CPEncoder<32,16> and the distance against its
    hamming_combined_scalar<32,16,2> (tests/golden/make_residual_golden.py)."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "residual_golden.npz"))
    x = g["x_%d" % dim]
    idx = residual_index(cp, dim, 32, 16, 2, conv=conv)
    idx.add_batch_parallel(x)
    words = idx.binary_codes()[:, 0]
    assert np.array_equal(words & np.uint64(0xFFFFFFFF), g["primary_%d_c%d" % (dim, conv)])
    assert np.array_equal(words >> np.uint64(32), g["residual_%d_c%d" % (dim, conv)])
    if dim == 128 and conv == 2:
        codes = idx.codes()
        assert np.array_equal(idx.code_distance(codes[:16], codes), g["combined_128_c2"].astype(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("Kp,R,shift,dim,M", [(32, 16, 2, 128, 16), (32, 32, 1, 100, 32), (16, 16, 3, 300, 8), (8, 4, 0, 64, 16),
                                              (64, 32, 2, 128, 16), (64, 16, 3, 200, 32)])  # the reference's K = 64 configurations
def test_residual_index_matches_oracle(cp, oracle, Kp, R, shift, dim, M):
    """Residual codes end to end: combined distance in the kNN graph, select_neighbors, the walk,
    brute force, incremental insertion and a save/load round trip."""
    n0, n1, K = 1800, 300, Kp + R
    base, q = synthetic.gaussian_mixture(n0 + n1, 25, dim, 8, 0.3, Kp * 100 + R)
    idx = residual_index(cp, dim, Kp, R, shift, M=M)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 8)
    assert idx.get_param("residual_bits") == R and idx.get_param("residual_shift") == shift
    idx.add_batch_parallel(base[:n0])
    signs = oracle.sign_tables(dim, K, 42)
    cb = 1 if idx.padded_dim <= 128 else 2
    codes = (oracle.encode(base, K, cb, signs, 2) & 1).astype(np.uint8)
    qcodes = (oracle.encode(q, K, cb, signs, 2) & 1).astype(np.uint8)
    assert np.array_equal(idx.codes(), codes[:n0])
    with oracle.residual_weighting(Kp, shift):
        assert np.array_equal(idx.code_distance(codes[:40], codes[:70]), oracle.code_distance(codes[:40], codes[:70]))
        knn_k = min(64, 2 * M)
        wn, wd = oracle.knn_graph(codes[:n0], knn_k)
        nbrs, dist = idx.knn_graph(codes[:n0], knn_k)
        assert np.array_equal(nbrs, wn) and np.array_equal(dist, wd)
        adj = oracle.select_neighbors(codes[:n0], wn, M, True)
        assert np.array_equal(idx.adjacency(), adj)
        entry = idx.entry_ids()
        ids, dd = idx.search_batch(q, 10, 80)
        wi, wdd = oracle.search_codes(qcodes, codes[:n0], adj, entry, 80, 10, n_seed=8)
        assert np.array_equal(ids, wi) and np.array_equal(dd, wdd)
        bi, bd = idx.brute_force_search_batch(q[:5], 15)
        full = oracle.code_distance(qcodes[:5], codes[:n0]).astype(np.int64)
        for qi in range(5):
            order = np.lexsort((np.arange(n0), full[qi]))[:15]
            assert np.array_equal(bi[qi], order.astype(np.uint32)) and np.array_equal(bd[qi], full[qi][order].astype(np.float32))
        # incremental insertion under the combined distance
        idx.add_batch(base[n0:])
        want = oracle_insert(oracle, codes, adj, n0, n1, M, True, 200, entry, 8)
        assert np.array_equal(idx.adjacency(), want)
    # both kNN kernels give the same lists; the bit-sliced one needs whole blocks of 8 components
    with oracle.residual_weighting(Kp, shift):
        wn, wd = oracle.knn_graph(codes, 70)
    for kern in (1, 2):
        idx.set_param("knn_kernel", kern)
        if kern == 2 and (K % 8 or Kp % 8):
            with pytest.raises(cp.CPHNSWError):
                idx.knn_graph(codes, 70)
            continue
        nbrs, dist = idx.knn_graph(codes, 70)
        assert np.array_equal(nbrs, wn) and np.array_equal(dist, wd)
    idx.set_param("knn_kernel", 0)
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "res.cphnsw")
        idx.save(path)
        again = cp.CPHNSWIndex.load(path)
        assert again.get_param("residual_bits") == R and again.get_param("residual_shift") == shift
        a, b = idx.search_batch(q, 5, 40), again.search_batch(q, 5, 40)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.gpu
def test_residual_parameters_are_validated(cp):
    idx = cp.CPHNSWIndex(128, K=32, M=16)
    with pytest.raises(ValueError):
        idx.set_param("residual_bits", 8)       # needs binary codes
    b = cp.CPHNSWIndex.binary(128, K=48, M=16)
    with pytest.raises(ValueError):
        b.set_param("residual_bits", 48)        # no primary part left
    with pytest.raises(ValueError):
        b.set_param("residual_bits", 15)        # primary part must fill whole words
    with pytest.raises(ValueError):
        b.set_param("residual_shift", 5)
    b.set_param("residual_bits", 16)
    with pytest.raises(ValueError):
        b.set_param("binary_codes", 0)

