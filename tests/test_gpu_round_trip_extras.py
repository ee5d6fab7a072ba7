"""GPU tests of the pieces around the hot path: rank-based pruning against the oracle, candidate ids that
name no node, the bounded-wait exit of the kNN kernels, the library's code-distance walk against the
reference's own walk, concurrent searches on one handle, installation from host buffers."""
import os
import threading

import numpy as np
import pytest

from cphnsw_b200 import synthetic

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF
WALK = np.load(os.path.join(os.path.dirname(__file__), "golden", "walk_golden.npz"))


def make_index(cp, dim, K=32, cb=1, M=32):
    return cp.CPHNSWIndex(dim, M=M, ef_construction=max(200, M), K=K, component_bytes=cb)


# ---- rank-based pruning ------------------------------------------------------------------------------
@pytest.mark.parametrize("n,k,M,alpha", [(1, 8, 4, 1.0), (40, 64, 32, 1.1), (700, 64, 32, 1.1), (1500, 32, 16, 1.0),
                                         (1500, 64, 32, 1.5), (900, 20, 32, 1.1), (2000, 64, 64, 3.0), (1200, 48, 8, 1.1)])
def test_rank_prune_matches_oracle(cp, oracle, n, k, M, alpha):
    base, _ = synthetic.gaussian_mixture(n, 1, 64, max(2, n // 200), 0.3, n + k)
    codes = oracle.encode(base, 32, 1, oracle.sign_tables(64, 32, 42))
    cand, _ = oracle.knn_graph(codes, k)
    idx = make_index(cp, 64, M=min(M, 64))
    got = idx.rank_prune(cand, M, alpha)
    want = oracle.rank_prune(cand, M, alpha)
    assert np.array_equal(got, want)
    valid = got != INVALID
    assert (got[valid] < n).all() and not (got == np.arange(n, dtype=np.uint32)[:, None]).any()
    s = np.sort(got, axis=1)
    assert not ((s[:, 1:] == s[:, :-1]) & (s[:, 1:] != INVALID)).any()  # each id once in a row


def test_rank_prune_build_matches_oracle_and_searches(cp, oracle):
    n, dim, K, M = 4000, 128, 32, 32
    base, q = synthetic.gaussian_mixture(n, 100, dim, 16, 0.3, 5)
    idx = make_index(cp, dim, K, 1, M)
    idx.set_param("entry_scan", 128)
    idx.set_param("rank_prune", 1)
    idx.set_param("rank_pruning_alpha", 1.1)
    idx.add_batch_parallel(base)
    codes = oracle.encode(base, K, 1, oracle.sign_tables(dim, K, 42))
    cand, _ = oracle.knn_graph(codes, 64)
    assert np.array_equal(idx.adjacency(), oracle.rank_prune(cand, M, 1.1))
    ids, _ = idx.search_and_rerank_batch(q, 10, 100, 200)
    gt = oracle.ground_truth(q, base, 10)
    assert oracle.recall_at_k(ids, gt, 10) > 0.8
    with pytest.raises(ValueError):
        idx.set_param("rank_pruning_alpha", 0.5)
    with pytest.raises(ValueError):
        idx.set_param("rank_pruning_alpha", 3.5)


# ---- ids that name no node are skipped, never read -----------------------------------------------------
def test_select_neighbors_skips_out_of_range_candidates(cp, oracle):
    n, k, M = 600, 32, 16
    base, _ = synthetic.gaussian_mixture(n, 1, 128, 4, 0.3, 9)
    codes = oracle.encode(base, 32, 1, oracle.sign_tables(128, 32, 42))
    cand, _ = oracle.knn_graph(codes, k)
    bad = cand.copy()
    rng = np.random.default_rng(1)
    for row in range(0, n, 3):  # a few ids >= n among the candidates, the largest legal-looking ones included
        for col in rng.choice(k, 3, replace=False):
            bad[row, col] = rng.choice([n, n + 7, 0x7FFFFFFF, 0xFFFFFFFE])
    idx = make_index(cp, 128, M=M)
    got = idx.select_neighbors(codes, bad, M, True)
    clean = np.where(bad >= n, INVALID, bad).astype(np.uint32)
    assert np.array_equal(got, oracle.select_neighbors(codes, clean, M, True))
    assert (got[got != INVALID] < n).all()


# ---- the bounded wait of the kNN kernels ----------------------------------------------------------------
@pytest.mark.parametrize("kernel", [1, 2])
def test_lost_wait_is_reported_and_the_handle_stays_usable(cp, oracle, kernel):
    # nothing is made to hang: the first wait of the launch is given zero polls, so it gives up at once,
    # the blocks let their copies in flight land (full poll limit) and return, the call reports the status
    n, k = 3000, 16
    base, _ = synthetic.gaussian_mixture(n, 1, 128, 8, 0.3, 3)
    codes = oracle.encode(base, 32, 1, oracle.sign_tables(128, 32, 42))
    idx = make_index(cp, 128)
    idx.set_param("knn_kernel", kernel)
    idx.set_param("first_wait_polls", 0)
    with pytest.raises(cp.CPHNSWError) as err:
        idx.knn_graph(codes, k)
    assert "[%d]" % cp.E_DEVICE_WAIT in str(err.value)
    idx.check_device_status()  # the status word was cleared by the failing call
    idx.set_param("first_wait_polls", 1 << 22)
    got, gd = idx.knn_graph(codes, k)
    want, wd = oracle.knn_graph(codes, k)
    assert np.array_equal(got, want) and np.array_equal(gd, wd)
    # a bulk build that loses its wait leaves the index as it was
    idx.add_batch_parallel(base[:1000])
    adj = idx.adjacency()
    idx.set_param("first_wait_polls", 0)
    with pytest.raises(cp.CPHNSWError):
        idx.add_batch_parallel(base[1000:2000])
    idx.set_param("first_wait_polls", 1 << 22)
    assert idx.size() == 1000 and np.array_equal(idx.adjacency(), adj)
    idx.add_batch_parallel(base[1000:2000])
    assert idx.size() == 2000


# ---- the code-distance walk against the reference's SearchEngine (tie-free cases: exact) --------------
def _entries(row):
    return row[row != INVALID]


def _entries_first(n, entry, adj):
    """Entry ids of an index are evenly spaced node ids; renumber the nodes so that the wanted entry
    points are exactly those.  Returns perm (perm[new] = old) and the renumbered adjacency."""
    ne = len(entry)
    slots = (np.arange(ne, dtype=np.uint64) * n // ne).astype(np.int64)
    rest = np.setdiff1d(np.arange(n), slots)
    perm = np.empty(n, np.uint32)
    perm[slots] = entry
    perm[rest] = np.setdiff1d(np.arange(n, dtype=np.uint32), entry)
    inv = np.empty(n, np.uint32)
    inv[perm] = np.arange(n, dtype=np.uint32)
    adj2 = np.where(adj[perm] == INVALID, INVALID, inv[np.minimum(adj[perm], n - 1)]).astype(np.uint32)
    return perm, adj2


def test_walk_equals_reference_walk_tie_free(cp, oracle):
    for c in range(WALK["tf64_q"].shape[0]):
        ef = int(WALK["tf64_ef"][c])
        codes = oracle.unpack_sign_bits(WALK["tf64_codes"][c], 64)
        q = oracle.unpack_sign_bits(WALK["tf64_q"][c:c + 1], 64)
        entry = _entries(WALK["tf64_entry"][c])
        n = codes.shape[0]
        perm, adj2 = _entries_first(n, entry, WALK["tf64_adj"][c])
        idx = cp.CPHNSWIndex.binary(64, M=6, ef_construction=200, K=64)
        idx.install(np.zeros((n, 64), np.float32), codes[perm], adj2)
        assert np.array_equal(idx.get_code(5), codes[perm][5])
        # the walk is seeded with exactly the reference's entry points: all scanned ids seed it
        idx.set_param("entry_scan", len(entry))
        idx.set_param("k_entry", len(entry))
        assert np.array_equal(perm[idx.entry_ids()], entry)
        ids, dist = idx.search_codes_batch(q, ef, ef)
        got = np.where(ids[0] == INVALID, INVALID, perm[np.minimum(ids[0], n - 1)])
        assert np.array_equal(got, WALK["tf64_ids"][c, :ef]), c
        assert np.array_equal(dist[0], WALK["tf64_dist"][c, :ef]), c


def test_walk_equals_reference_walk_residual_tie_free(cp, oracle):
    for c in range(WALK["tfr_qp"].shape[0]):
        ef = int(WALK["tfr_ef"][c])
        codes = np.concatenate([oracle.unpack_sign_bits(WALK["tfr_prim"][c], 32), oracle.unpack_sign_bits(WALK["tfr_resi"][c], 16)], axis=1)
        q = np.concatenate([oracle.unpack_sign_bits(WALK["tfr_qp"][c:c + 1], 32), oracle.unpack_sign_bits(WALK["tfr_qr"][c:c + 1], 16)], axis=1)
        entry = _entries(WALK["tfr_entry"][c])
        n = codes.shape[0]
        adj = WALK["tfr_adj"][c]
        perm, adj2 = _entries_first(n, entry, adj)
        idx = cp.CPHNSWIndex.binary(64, M=6, ef_construction=200, K=48)
        idx.set_param("residual_bits", 16)
        idx.set_param("residual_shift", 2)
        idx.install(np.zeros((n, 64), np.float32), codes[perm], adj2)
        idx.set_param("entry_scan", len(entry))
        idx.set_param("k_entry", len(entry))
        ids, dist = idx.search_codes_batch(q, ef, ef)
        got = np.where(ids[0] == INVALID, INVALID, perm[np.minimum(ids[0], n - 1)])
        assert np.array_equal(got, WALK["tfr_ids"][c, :ef]), c
        assert np.array_equal(dist[0], WALK["tfr_dist"][c, :ef]), c


# ---- concurrent searches on one handle -------------------------------------------------------------------
def test_concurrent_single_query_searches_equal_the_batch(cp):
    # the reference's callers search from OpenMP loops, one query per call (evaluation/eval_sift.cpp:380-387)
    n, nq, dim = 20000, 256, 128
    base, q = synthetic.gaussian_mixture(n, nq, dim, 40, 0.3, 21)
    idx = make_index(cp, dim)
    idx.set_param("entry_scan", 512)
    idx.set_param("k_entry", 8)
    idx.add_batch_parallel(base)
    want_i, want_d = idx.search_and_rerank_batch(q, 10, 100, 200)
    ws_i, ws_d = idx.search_batch(q, 10, 64)
    got_i = np.zeros_like(want_i)
    got_d = np.zeros_like(want_d)
    gs_i = np.zeros_like(ws_i)
    gs_d = np.zeros_like(ws_d)
    errors = []

    def worker(t, nthreads):
        try:
            for i in range(t, nq, nthreads):
                a, b = idx.search_and_rerank_batch(q[i:i + 1], 10, 100, 200)
                got_i[i], got_d[i] = a[0], b[0]
                a, b = idx.search_batch(q[i:i + 1], 10, 64)
                gs_i[i], gs_d[i] = a[0], b[0]
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(t, 16)) for t in range(16)]
    for t in threads:
        t.start()
    # a large batch takes its turn on the wide context while the single-query calls run
    big_i, big_d = idx.search_and_rerank_batch(q, 10, 100, 200)
    for t in threads:
        t.join()
    assert not errors, errors
    assert np.array_equal(got_i, want_i) and np.array_equal(got_d, want_d)
    assert np.array_equal(gs_i, ws_i) and np.array_equal(gs_d, ws_d)
    assert np.array_equal(big_i, want_i) and np.array_equal(big_d, want_d)


def test_narrow_launch_equals_wide_launch(cp):
    # up to 32 queries run one block per query, more fill the GPU: same results either way
    n, dim = 12000, 96
    base, q = synthetic.gaussian_mixture(n, 200, dim, 24, 0.3, 4)
    for kern in (1, 2):
        idx = make_index(cp, dim)
        idx.set_param("entry_scan", 256)
        idx.set_param("search_kernel", kern)
        idx.add_batch_parallel(base)
        wide = idx.search_and_rerank_batch(q, 10, 80, 150, want_stats=True)
        for lo, hi in ((0, 1), (1, 33), (33, 40), (40, 72)):
            part = idx.search_and_rerank_batch(q[lo:hi], 10, 80, 150, want_stats=True)
            assert all(np.array_equal(a, b[lo:hi]) for a, b in zip(part, wide))
        mp = idx.search_multiprobe_batch(q[:64], 10, 50, 4)
        one = idx.search_multiprobe_batch(q[3:4], 10, 50, 4)
        assert np.array_equal(one[0][0], mp[0][3]) and np.array_equal(one[1][0], mp[1][3])


def test_binary_codes_cannot_be_switched_off_when_components_would_not_fit(cp):
    # a binary-code handle keeps one byte per component whatever the dimension; full (index, sign) components
    # of padded dim 512 do not fit a byte, so switching the mode off must be refused, not silently truncate
    idx = cp.CPHNSWIndex.binary(300, K=32)
    with pytest.raises(ValueError):
        idx.set_param("binary_codes", 0)
    assert idx.get_param("binary_codes") == 1
    small = cp.CPHNSWIndex.binary(100, K=32)  # padded dim 128 fits a byte: allowed
    small.set_param("binary_codes", 0)
    assert small.get_param("binary_codes") == 0


def test_installed_adjacency_with_foreign_ids_is_searched_safely(cp, oracle):
    # rows installed from outside may hold ids that name no node: every kernel treats them as "no node"
    n, M = 2000, 32
    base, q = synthetic.gaussian_mixture(n, 50, 128, 8, 0.3, 12)
    ref = make_index(cp, 128)
    ref.set_param("entry_scan", 64)
    ref.add_batch_parallel(base)
    codes, adj = ref.codes(), ref.adjacency()
    bad = adj.copy()
    bad[::7, 5] = n + 11
    bad[3::11, 0] = 0xFFFFFFFE
    idx = make_index(cp, 128)
    idx.set_param("entry_scan", 64)
    idx.install(base, codes, bad)
    clean = np.where(bad >= n, INVALID, bad).astype(np.uint32)
    _, rot, _ = oracle.encode(q, 32, 1, oracle.sign_tables(128, 32, 42), 2, want_rotated=True)
    want = oracle.search(rot, codes, clean, idx.entry_ids(), 100, 10, n_seed=4)
    got = idx.search_batch(q, 10, 100)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    assert idx.verify_connectivity() == oracle.connectivity(clean, idx.entry_ids())
    more, _ = synthetic.gaussian_mixture(300, 1, 128, 8, 0.3, 13)
    idx.add_batch(more)  # the reverse-edge pass reads the installed rows
    assert idx.size() == n + 300 and (idx.adjacency()[n:] < n + 300).all()


# ---- links chosen on the fp32 vectors ("exact_edges": the legacy hybrid construction) ---------------------------
@pytest.mark.parametrize("n,dim,M,knn_k,keep", [(2500, 128, 32, 64, True), (1800, 96, 16, 32, True), (900, 40, 32, 64, False),
                                                (1200, 200, 8, 20, True), (60, 128, 32, 64, True)])
def test_exact_edges_build_matches_oracle(cp, oracle, n, dim, M, knn_k, keep):
    base, q = synthetic.gaussian_sphere(n, 40, dim, n + M)
    base[7] = base[3]  # exact duplicates: equal distances, ties by id
    base[8] = base[3]
    idx = cp.CPHNSWIndex(dim, M=M, ef_construction=200, K=32, component_bytes=2 if dim > 128 else 1)
    idx.set_param("exact_edges", 1)
    idx.set_param("knn_k", knn_k)
    idx.set_param("keep_pruned", int(keep))
    idx.set_param("entry_scan", min(n, 64))
    idx.add_batch_parallel(base)
    k = max(M, min(knn_k, 64))
    cand = oracle.exact_candidates(base, k)
    assert np.array_equal(idx.adjacency(), oracle.select_neighbors_exact(base, cand, M, keep))
    ids, _ = idx.search_and_rerank_batch(q, 10, 100, 100)
    assert (ids[ids != INVALID] < n).all()
    # "prune" = 0: the M exact nearest are the links
    cut = cp.CPHNSWIndex(dim, M=M, ef_construction=200, K=32, component_bytes=2 if dim > 128 else 1)
    cut.set_param("exact_edges", 1)
    cut.set_param("prune", 0)
    cut.add_batch_parallel(base)
    assert np.array_equal(cut.adjacency(), oracle.exact_candidates(base, M))


def test_exact_edges_lift_recall_on_unclustered_data(cp, oracle):
    # on vectors without cluster structure the code-distance kNN graph navigates poorly; exact links let the walk
    # reach what the code can rank
    base, q = synthetic.gaussian_sphere(30000, 300, 128, 5)
    gt = oracle.ground_truth(q, base, 10)
    rec = {}
    for exact in (0, 1):
        idx = make_index(cp, 128)
        idx.set_param("exact_edges", exact)
        idx.add_batch_parallel(base)
        ids, _ = idx.search_and_rerank_batch(q, 10, 500, 500)
        rec[exact] = oracle.recall_at_k(ids, gt, 10)
    assert rec[1] > rec[0] + 0.1 and rec[1] > 0.8, rec


@pytest.mark.parametrize("kernel,K", [(0, 32), (1, 32), (0, 64)])
def test_beams_wider_than_1024_match_oracle(cp, oracle, kernel, K):
    # the two-warp kernel's tiered W: 32 buckets up to 1,024, 64 buckets (two per lane) up to 2,048; beyond that, and when
    # asked for, the one-warp kernel's flat W (three-level rank search)
    n, dim, M = 6000, 128, 32
    base, q = synthetic.gaussian_mixture(n, 24, dim, 6, 0.3, 17)
    idx = make_index(cp, dim, K, 1, M)
    idx.set_param("search_kernel", kernel)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 8)
    idx.add_batch_parallel(base)
    signs = oracle.sign_tables(dim, K, 42)
    codes, adj = idx.codes(), idx.adjacency()
    _, rot, _ = oracle.encode(q, K, 1, signs, 2, want_rotated=True)
    for k, ef in ((10, 1025), (100, 1500), (10, 2047), (10, 2048), (2000, 2000), (50, 4096)):
        ids, dist, stats = idx.search_batch(q, k, ef, want_stats=True)
        wi, wd, ws = oracle.search(rot, codes, adj, idx.entry_ids(), max(ef, k), k, want_stats=True, n_seed=8)
        assert np.array_equal(ids, wi) and np.array_equal(dist, wd) and np.array_equal(stats, ws), (k, ef)
    ids, dist = idx.search_and_rerank_batch(q, 10, 100, 3000)
    cand, _ = oracle.search(rot, codes, adj, idx.entry_ids(), 3000, 3000, n_seed=8)
    wi, wd = oracle.rerank(q, base, cand, 10)
    assert np.allclose(dist, wd, rtol=1e-5, atol=1e-6) and (ids == wi).mean() > 0.99
    with pytest.raises(ValueError):
        idx.search_batch(q, 10, 4097)


def test_binary_mode_stores_packed_sign_bits(cp, oracle, tmp_path):
    """Binary-code mode keeps a node's code as packed sign bits between build stages (8 times smaller than one byte per
    bit); accessors, insertion, the index file and the walk give what the byte form gave."""
    n, dim, K, M = 5000, 128, 64, 16
    base, q = synthetic.gaussian_mixture(n + 700, 40, dim, 10, 0.3, 5)
    plain = make_index(cp, dim, 32, 1, M)
    plain.add_batch_parallel(base[:n])
    assert plain.get_param("stored_code_bytes") == 32            # full components: one byte each
    idx = cp.CPHNSWIndex.binary(dim, K=K, M=M)
    idx.set_param("entry_scan", 64)
    idx.set_param("k_entry", 8)
    idx.add_batch_parallel(base[:n])
    assert idx.get_param("stored_code_bytes") == K // 8         # 64 sign bits in two words
    signs = oracle.sign_tables(dim, K, 42)
    want = oracle.encode(base[:n + 700], K, 1, signs, 2) & 1
    codes = idx.codes()
    assert codes.shape == (n, K) and np.array_equal(codes, want[:n])
    assert np.array_equal(idx.get_code(4321), want[4321])
    assert np.array_equal(idx.binary_codes()[:, 0], oracle.pack_sign_bits(want[:n]))
    ids0, d0, st0 = idx.search_batch(q, 10, 100, want_stats=True)
    wi, wd = oracle.search_codes(oracle.encode(q, K, 1, signs, 2) & 1, want[:n], idx.adjacency(), idx.entry_ids(), 100, 10, n_seed=8)
    assert np.array_equal(ids0, wi) and np.array_equal(d0, wd)
    path = str(tmp_path / "binary.cph")
    idx.save(path)
    back = cp.CPHNSWIndex.load(path)
    assert back.get_param("stored_code_bytes") == K // 8
    assert np.array_equal(back.codes(), codes)
    ids1, d1, st1 = back.search_batch(q, 10, 100, want_stats=True)
    assert np.array_equal(ids1, ids0) and np.array_equal(d1, d0) and np.array_equal(st1, st0)
    # insertion unpacks, extends and packs again
    idx.add_batch(base[n:])
    back.add_batch(base[n:])
    assert idx.size() == n + 700 and idx.get_param("stored_code_bytes") == K // 8
    assert np.array_equal(idx.codes(), want) and np.array_equal(idx.adjacency(), back.adjacency())
    a = idx.search_and_rerank_batch(q, 10, 100, 300)
    b = back.search_and_rerank_batch(q, 10, 100, 300)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
