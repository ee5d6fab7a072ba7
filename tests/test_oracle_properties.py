"""Properties of the oracle's distance / kNN / select_neighbors / search / rerank restatements,
cross-checked against independent numpy formulations (the reference's legacy sources for these
are absent, so these pin the oracle's own definitions)."""
import numpy as np
import pytest

from cphnsw_b200 import synthetic

INVALID = 0xFFFFFFFF


def small_index(oracle, n=600, nq=20, dim=32, K=16, seed=3, cb=1):
    base, q = synthetic.gaussian_mixture(n, nq, dim, 6, 0.3, seed)
    signs = oracle.sign_tables(dim, K, 42)
    codes = oracle.encode(base, K, cb, signs)
    return base, q, signs, codes


def tree_score(terms):
    """Sum of K term arrays in the oracle's declared order: blocks of 32, pairs 16/8/4/2/1 apart."""
    K = len(terms)
    zero = np.zeros_like(terms[0])
    score = zero.copy()
    for c0 in range(0, K, 32):
        t = [terms[c0 + j] if c0 + j < K else zero for j in range(32)]
        step = 16
        while step >= 1:
            for j in range(step):
                t[j] = (t[j] + t[j + step]).astype(np.float32)
            step //= 2
        score = (score + t[0]).astype(np.float32)
    return score


def test_code_distance_counts_differing_components(oracle):
    rng = np.random.default_rng(0)
    for dt in (np.uint8, np.uint16):
        a = rng.integers(0, 6, (17, 32)).astype(dt)
        b = rng.integers(0, 6, (23, 32)).astype(dt)
        want = (a[:, None, :] != b[None, :, :]).sum(-1).astype(np.uint16)
        assert np.array_equal(oracle.code_distance(a, b), want)
    # identical code -> 0 (evaluation/debug_code_storage.cpp:63-105)
    assert (np.diag(oracle.code_distance(a, a)) == 0).all()


def test_knn_graph_against_full_sort(oracle):
    base, q, signs, codes = small_index(oracle)
    n = codes.shape[0]
    k = 10
    nbrs, dist = oracle.knn_graph(codes, k)
    D = oracle.code_distance(codes, codes).astype(np.int64)
    for i in range(n):
        order = sorted((int(D[i, j]), j) for j in range(n) if j != i)[:k]
        assert nbrs[i].tolist() == [j for _, j in order]
        assert dist[i].tolist() == [d for d, _ in order]
    assert not (nbrs == np.arange(n)[:, None]).any()  # no self loops (evaluation/debug_gpu_knn.cpp:42-68)
    # row-range form returns the same rows
    part, _ = oracle.knn_graph(codes, k, 100, 164)
    assert np.array_equal(part, nbrs[100:164])


def test_knn_graph_pads_small_inputs(oracle):
    codes = np.random.default_rng(1).integers(0, 4, (5, 8)).astype(np.uint8)
    nbrs, dist = oracle.knn_graph(codes, 8)
    assert (nbrs[:, 4:] == INVALID).all() and (dist[:, 4:] == 0xFFFF).all()
    assert (np.sort(nbrs[:, :4], axis=1) == np.array([[j for j in range(5) if j != i] for i in range(5)])).all()


def select_py(codes, i, cand, M, keep):
    def d(a, b):
        return int((codes[a] != codes[b]).sum())
    R, Wd = [], []
    for e in cand:
        if len(R) >= M:
            break
        if e == INVALID:
            continue
        (R if all(d(e, i) < d(e, r) for r in R) else Wd).append(int(e))
    if keep:
        R += Wd[: max(0, M - len(R))]
    return R + [INVALID] * (M - len(R))


@pytest.mark.parametrize("keep", [True, False])
def test_select_neighbors_matches_python(oracle, keep):
    base, q, signs, codes = small_index(oracle, n=300)
    nbrs, _ = oracle.knn_graph(codes, 24)
    nbrs[5, 20:] = INVALID
    adj = oracle.select_neighbors(codes, nbrs, 12, keep)
    for i in range(codes.shape[0]):
        assert adj[i].tolist() == select_py(codes, i, nbrs[i], 12, keep), i
    if keep:  # with k <= M nothing is dropped, only reordered
        adj2 = oracle.select_neighbors(codes, nbrs, 24, True)
        assert np.array_equal(np.sort(adj2, axis=1), np.sort(nbrs, axis=1))


def test_search_is_exhaustive_when_beam_covers_component(oracle):
    """With ef >= n and a connected graph the walk visits everything, so it must return the exact
    top-k under the asymmetric score; results are ascending (evaluation/qa_protocol.cpp:116-166)."""
    base, q, signs, codes = small_index(oracle, n=400, dim=32, K=16)
    n = codes.shape[0]
    _, rot, _ = oracle.encode(q, 16, 1, signs, want_rotated=True)
    # ring + kNN edges: connected
    nbrs, _ = oracle.knn_graph(codes, 7)
    adj = np.concatenate([nbrs, ((np.arange(n) + 1) % n)[:, None].astype(np.uint32)], axis=1)
    ids, dist = oracle.search(rot, codes, adj, np.array([0], np.uint32), n, 10)
    P = rot.shape[2]
    for qi in range(q.shape[0]):
        terms = []
        for r in range(16):
            v = rot[qi, r, codes[:, r] >> 1]
            terms.append(np.where(codes[:, r] & 1, -v, v).astype(np.float32))
        score = tree_score(terms)
        # the declared tree order stays within 1e-5 relative of the reference's sequential sum
        seq = np.zeros(n, np.float32)
        for tm in terms:
            seq = (seq + tm).astype(np.float32)
        assert np.allclose(score, seq, rtol=1e-5, atol=1e-5 * float(np.abs(np.stack(terms)).sum(0).max()))
        order = sorted((float(-score[j]), j) for j in range(n))[:10]
        assert ids[qi].tolist() == [j for _, j in order]
        assert np.array_equal(dist[qi], np.array([d for d, _ in order], np.float32))
        assert (np.diff(dist[qi]) >= 0).all()


def test_identity_query_scores_sum_of_magnitudes(oracle):
    # Score(X, Code_X) = sum of winning magnitudes (evaluation/debug_estimator.cpp:74-82)
    base, q, signs, codes = small_index(oracle, n=50)
    c, rot, mag = oracle.encode(base[:5], 16, 1, signs, want_rotated=True)
    for i in range(5):
        s = np.float32(0)
        for r in range(16):
            v = rot[i, r, c[i, r] >> 1]
            s = np.float32(s + (-v if c[i, r] & 1 else v))
        assert np.isclose(s, mag[i].sum(), rtol=1e-5)


def test_recall_non_decreasing_in_beam_and_rerank_orders(oracle):
    base, q, signs, codes = small_index(oracle, n=2000, nq=40, dim=64, K=16)
    _, rot, _ = oracle.encode(q, 16, 1, signs, want_rotated=True)
    nbrs, _ = oracle.knn_graph(codes, 32)
    adj = oracle.select_neighbors(codes, nbrs, 16)
    entry = (np.arange(64) * 2000 // 64).astype(np.uint32)
    gt = oracle.ground_truth(q, base, 10)
    last = -1.0
    for ef in (20, 80, 320):  # evaluation/qa_protocol.cpp:559-640
        ids, _ = oracle.search(rot, codes, adj, entry, ef, ef)
        rid, rd = oracle.rerank(q, base, ids, 10)
        r = oracle.recall_at_k(rid, gt, 10)
        assert r >= last - 1e-9
        last = r
        assert (np.diff(rd, axis=1) >= 0).all()
        # reranked distance is -<q,x>
        for qi in range(3):
            assert np.allclose(rd[qi], -(base[rid[qi]] @ q[qi]), rtol=1e-5, atol=1e-6)
    assert last > 0.5


def test_zero_vector_and_duplicates_do_not_break(oracle):
    # evaluation/qa_protocol.cpp:409-553: N < batch, duplicates, zero vector -> no NaN
    dim, K = 16, 8
    x = np.zeros((4, dim), np.float32)
    x[1, 0] = 1.0
    x[2] = x[1]
    signs = oracle.sign_tables(dim, K, 42)
    codes, rot, mag = oracle.encode(x, K, 1, signs, want_rotated=True)
    assert (codes[0] == 0).all()  # all-zero rotation: index 0, positive
    assert np.array_equal(codes[1], codes[2])
    assert np.isfinite(rot).all()


def test_probe_sequence_matches_exhaustive_enumeration(oracle):
    """The multiprobe sequence must be the T cheapest rank combinations in ascending cost
    (resources/cross-polytope-lsh/consolidated.tex:391-425), the primary code first."""
    import itertools
    rng = np.random.default_rng(5)
    K, P, T = 3, 8, 12
    rot = rng.standard_normal((6, K, P)).astype(np.float32)
    pc = oracle.probe_codes(rot, 1, T)
    V = min(P, T + 1)
    for q in range(rot.shape[0]):
        order = [sorted(range(P), key=lambda i: (-abs(rot[q, r, i]), i)) for r in range(K)]
        cost = [[np.float32(np.float32(abs(rot[q, r, order[r][0]]) - abs(rot[q, r, order[r][v]])) ** 2) for v in range(V)]
                for r in range(K)]
        states = []
        for rk in itertools.product(range(V), repeat=K):
            s = np.float32(0)
            for r in range(K):
                if rk[r]:
                    s = np.float32(s + cost[r][rk[r]])
            states.append((float(s), rk))
        states.sort()
        for t in range(T):
            rk = states[t][1]
            want = [(order[r][rk[r]] << 1) | int(rot[q, r, order[r][rk[r]]] < 0) for r in range(K)]
            assert pc[q, t].tolist() == want, (q, t)
    # probe 0 is the ordinary code of the query
    assert np.array_equal(pc[:, 0, :] >> 1, np.abs(rot).argmax(axis=2))


def test_multiprobe_merge_and_monotone_recall(oracle):
    base, q, signs, codes = small_index(oracle, n=1500, nq=30, dim=64, K=16)
    _, rot, _ = oracle.encode(q, 16, 1, signs, want_rotated=True)
    nbrs, _ = oracle.knn_graph(codes, 32)
    adj = oracle.select_neighbors(codes, nbrs, 16)
    entry = (np.arange(64) * 1500 // 64).astype(np.uint32)
    one_i, one_d = oracle.search_multiprobe(rot, 1, codes, adj, entry, 40, 10, 1, n_seed=8)
    qc = oracle.encode(q, 16, 1, signs)
    ref_i, ref_d = oracle.search_codes(qc, codes, adj, entry, 40, 10, n_seed=8)
    assert np.array_equal(one_i, ref_i) and np.array_equal(one_d, ref_d)  # one probe = plain symmetric search
    many_i, many_d = oracle.search_multiprobe(rot, 1, codes, adj, entry, 40, 10, 8, n_seed=8)
    assert (np.diff(many_d, axis=1) >= 0).all()
    for row in many_i:
        valid = row[row != 0xFFFFFFFF]
        assert len(set(valid.tolist())) == len(valid)  # every id once
    # distances are code distances to SOME probe, so they can only improve on the single-probe answer
    assert (many_d[:, 0] <= one_d[:, 0]).all()


# ---- diagnostics ------------------------------------------------------------------------------------------
def test_brute_force_is_the_sorted_prefix_of_all_scores(oracle):
    rng = np.random.default_rng(5)
    base = rng.standard_normal((400, 64)).astype(np.float32)
    q = rng.standard_normal((6, 64)).astype(np.float32)
    signs = oracle.sign_tables(64, 16, 42)
    codes = oracle.encode(base, 16, 1, signs, 2)
    _, rot, _ = oracle.encode(q, 16, 1, signs, 2, want_rotated=True)
    ids, dist = oracle.brute_force(rot, codes, 400)  # everything, ascending by (score, id)
    assert all(sorted(r.tolist()) == list(range(400)) for r in ids)
    key = [list(zip(d.tolist(), i.tolist())) for d, i in zip(dist, ids)]
    assert all(k == sorted(k) for k in key)
    top, _ = oracle.brute_force(rot, codes, 7)
    assert np.array_equal(top, ids[:, :7])
    over, od = oracle.brute_force(rot, codes[:3], 5)  # k > n pads
    assert (over[:, 3:] == 0xFFFFFFFF).all() and np.isinf(od[:, 3:]).all()


def test_linear_fit_and_calibration_pairs(oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal(500).astype(np.float32)
    y = (0.37 * x - 1.25 + 0.05 * rng.standard_normal(500)).astype(np.float32)
    a, b, r2 = oracle.linear_fit(x, y)
    pa, pb = np.polyfit(x.astype(np.float64), y.astype(np.float64), 1)
    assert np.isclose(a, pa, rtol=1e-9) and np.isclose(b, pb, rtol=1e-9)
    assert np.isclose(r2, np.corrcoef(x, y)[0, 1] ** 2, rtol=1e-9)
    assert oracle.linear_fit(np.ones(10, np.float32), y[:10]) == (0.0, float(np.float64(y[:10].astype(np.float64).mean())), 0.0)
    u, v = oracle.calibration_pairs(1000, 64, 42)
    u2, v2 = oracle.calibration_pairs(1000, 64, 42)
    assert np.array_equal(u, u2) and np.array_equal(v, v2) and u.max() < 1000 and v.max() < 1000
    assert not np.array_equal(u, oracle.calibration_pairs(1000, 64, 43)[0])


def test_calibration_has_positive_slope_on_clustered_data(oracle):
    rng = np.random.default_rng(1)
    centres = rng.standard_normal((8, 128)).astype(np.float32)
    base = centres[rng.integers(0, 8, 1500)] + 0.3 * rng.standard_normal((1500, 128)).astype(np.float32)
    base /= np.linalg.norm(base, axis=1, keepdims=True)
    signs = oracle.sign_tables(128, 32, 42)
    codes = oracle.encode(base, 32, 1, signs, 2)
    a, b, r2, x, y = oracle.calibrate(base, codes, signs, 32, 1, 2, 1000, 42)
    assert a > 0 and r2 > 0.5 and x.shape == (1000,) and (y >= -1.0001).all() and (y <= 1.0001).all()


def test_connectivity_counts_reachable_nodes(oracle):
    inv = 0xFFFFFFFF
    adj = np.array([[1, inv], [2, 0], [inv, inv], [4, inv], [3, 3], [0, inv]], np.uint32)  # {0,1,2} <- 5, {3,4} island
    assert oracle.connectivity(adj, np.array([0], np.uint32)) == 3
    assert oracle.connectivity(adj, np.array([5], np.uint32)) == 4
    assert oracle.connectivity(adj, np.array([3, 0, 0], np.uint32)) == 5
    assert oracle.connectivity(adj, np.array([], np.uint32)) == 0
    assert oracle.connectivity(adj, np.array([2, inv], np.uint32)) == 1



def rank_prune_py(cand, M, alpha):
    """Rank-based pruning written from the paper's text with Python sets and lists (1-based ranks)."""
    n, k = cand.shape
    lists = [[int(v) for v in row if v < n] for row in cand]
    pos = [{y: j + 1 for j, y in enumerate(row) if y < n} for row in cand.tolist()]
    kept = []
    for x in range(n):
        scored = []
        for y, ry in pos[x].items():
            detours = sum(1 for z, rz in pos[x].items()
                          if y in pos[z] and np.float32(alpha) * np.float32(max(rz, pos[z][y])) < np.float32(ry))
            scored.append((detours, ry, y))
        kept.append([y for _, _, y in sorted(scored)[:M]])
    rev = [[] for _ in range(n)]
    for x in range(n):
        for r, p in enumerate(kept[x]):
            rev[p].append((r, x))
    out = np.full((n, M), INVALID, np.uint32)
    for p in range(n):
        a, b = list(kept[p]), [x for _, x in sorted(rev[p])[:M]]
        row, turn = [], 0
        while len(row) < M:
            a = [v for v in a if v not in row]
            b = [v for v in b if v not in row]
            if not a and not b:
                break
            src = a if (not b or (a and turn == 0)) else b
            row.append(src.pop(0))
            turn ^= 1
        out[p, :len(row)] = row
    return out


@pytest.mark.parametrize("alpha", [1.0, 1.1, 2.0])
def test_rank_prune_matches_python(oracle, alpha):
    base, q, signs, codes = small_index(oracle, n=260)
    cand, _ = oracle.knn_graph(codes, 20)
    cand[7, 15:] = INVALID
    for M in (8, 20, 32):
        assert np.array_equal(oracle.rank_prune(cand, M, alpha), rank_prune_py(cand, M, alpha)), M
    # alpha = 1 is the paper's condition max(rank_XZ, rank_ZY) < rank_XY; a larger alpha can only remove detours,
    # so the nearest candidate (rank 1, never detourable) is always kept first
    adj = oracle.rank_prune(cand, 8, alpha)
    assert np.array_equal(adj[:, 0], cand[:, 0])
