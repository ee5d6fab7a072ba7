"""Generates tests/golden/walk_golden.npz from the REFERENCE's own graph walk,
SearchEngine<Policy>::search (include/cphnsw/search/search_engine.hpp:86-193), run over its
FlatGraph through oracle/ref_search_shim.cpp.

Two families of seeded cases:

* tie-free: a graph whose nodes all lie at DIFFERENT distances from the query (node i = the query
  code with i chosen bits flipped, ids shuffled; for the <32,16,2> residual code, every pair
  (h_primary, h_residual < 4) once).  The reference orders its heaps on `distance` alone
  (types.hpp:351-357), so only without ties is its result independent of heap internals; there the
  walk of the oracle and of the library must return exactly the reference's W.
* with ties: codes of clustered vectors; the reference's result is recorded for comparison in
  aggregate (distances tie massively under a 64-bit Hamming metric).

Run where the reference checkout is available:

    make -C oracle ref REF=<reference checkout> && python tests/golden/make_walk_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
sys.path.insert(0, os.path.join(HERE, "..", "..", "sparse-text-kmeans_b200"))
import oracle as O  # noqa: E402

EFS = (1, 2, 3, 5, 8, 16, 33, 65)


def random_adjacency(rng, n, M):
    adj = np.full((n, M), 0xFFFFFFFF, np.uint32)
    for i in range(n):
        deg = int(rng.integers(1, M + 1))
        others = np.delete(np.arange(n), i)
        adj[i, :deg] = rng.choice(others, size=deg, replace=False)
    return adj


def flip_code(q, bits):
    c = np.uint64(q)
    for b in bits:
        c ^= np.uint64(1) << np.uint64(b)
    return c


def main():
    R = O.RefSearch()
    rng = np.random.default_rng(20240)
    out = {}
    # ---- tie-free, 64 primary bits: 65 nodes at distances 0..64
    cases, n, M = 48, 65, 6
    codes = np.empty((cases, n), np.uint64)
    q = rng.integers(0, 2**63, size=cases, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=cases, dtype=np.uint64)
    adj = np.empty((cases, n, M), np.uint32)
    entry = np.full((cases, 3), 0xFFFFFFFF, np.uint32)
    ef = np.empty(cases, np.uint32)
    ids = np.full((cases, n), 0xFFFFFFFF, np.uint32)
    dist = np.full((cases, n), np.inf, np.float32)
    cnt = np.empty(cases, np.uint32)
    for c in range(cases):
        perm = rng.permutation(64)
        where = rng.permutation(n)  # node id of the code at distance i
        for i in range(n):
            codes[c, where[i]] = flip_code(q[c], perm[:i])
        adj[c] = random_adjacency(rng, n, M)
        ef[c] = EFS[c % len(EFS)]
        ne = min(int(rng.integers(1, 4)), int(ef[c]))  # the reference seeds W with every entry, bounded or not
        entry[c, :ne] = rng.choice(n, size=ne, replace=False)
        i_, d_, c_ = R.search_64(codes[c], adj[c], q[c:c + 1], entry[c, :ne], int(ef[c]))
        ids[c, :ef[c]], dist[c, :ef[c]], cnt[c] = i_[0], d_[0], c_[0]
    out.update(tf64_codes=codes, tf64_q=q, tf64_adj=adj, tf64_entry=entry, tf64_ef=ef, tf64_ids=ids, tf64_dist=dist,
               tf64_count=cnt)
    # ---- tie-free, <32,16,2>: distance (h_p << 2) + h_r with h_r < 4 -> 33 * 4 = 132 distinct values
    cases, n, M = 24, 132, 6
    prim = np.empty((cases, n), np.uint64)
    resi = np.empty((cases, n), np.uint64)
    qp = rng.integers(0, 2**32, size=cases, dtype=np.uint64)
    qr = rng.integers(0, 2**16, size=cases, dtype=np.uint64)
    adj = np.empty((cases, n, M), np.uint32)
    entry = np.full((cases, 3), 0xFFFFFFFF, np.uint32)
    ef = np.empty(cases, np.uint32)
    ids = np.full((cases, n), 0xFFFFFFFF, np.uint32)
    dist = np.full((cases, n), np.inf, np.float32)
    cnt = np.empty(cases, np.uint32)
    for c in range(cases):
        pp, pr = rng.permutation(32), rng.permutation(16)
        where = rng.permutation(n)
        for hp in range(33):
            for hr in range(4):
                prim[c, where[hp * 4 + hr]] = flip_code(qp[c], pp[:hp])
                resi[c, where[hp * 4 + hr]] = flip_code(qr[c], pr[:hr])
        adj[c] = random_adjacency(rng, n, M)
        ef[c] = (1, 4, 10, 40, 132)[c % 5]
        ne = min(int(rng.integers(1, 4)), int(ef[c]))
        entry[c, :ne] = rng.choice(n, size=ne, replace=False)
        i_, d_, c_ = R.search_32_16_s2(prim[c], resi[c], adj[c], qp[c:c + 1], qr[c:c + 1], entry[c, :ne], int(ef[c]))
        ids[c, :ef[c]], dist[c, :ef[c]], cnt[c] = i_[0], d_[0], c_[0]
    out.update(tfr_prim=prim, tfr_resi=resi, tfr_qp=qp, tfr_qr=qr, tfr_adj=adj, tfr_entry=entry, tfr_ef=ef, tfr_ids=ids,
               tfr_dist=dist, tfr_count=cnt)
    # ---- with ties: sign codes of clustered vectors, pruned kNN graph of the oracle
    from cphnsw_b200 import synthetic
    n, nq, dim, K, M, efv = 3000, 64, 64, 64, 32, 100
    base, qv = synthetic.gaussian_mixture(n, nq, dim, 12, 0.3, 7)
    signs = O.sign_tables(dim, K, 42)
    cb = (O.encode(base, K, 1, signs, O.FHT_AVX512) & 1).astype(np.uint8)
    cq = (O.encode(qv, K, 1, signs, O.FHT_AVX512) & 1).astype(np.uint8)
    cand, _ = O.knn_graph(cb, 64)
    adj = O.select_neighbors(cb, cand, M, True)
    entry = np.array([i * n // 8 for i in range(8)], np.uint32)
    i_, d_, c_ = R.search_64(O.pack_sign_bits(cb), adj, O.pack_sign_bits(cq), entry, efv)
    out.update(tie_codes=O.pack_sign_bits(cb), tie_q=O.pack_sign_bits(cq), tie_adj=adj, tie_entry=entry,
               tie_ef=np.uint32(efv), tie_ids=i_, tie_dist=d_)
    np.savez_compressed(os.path.join(HERE, "walk_golden.npz"), **out)
    print("wrote walk_golden.npz")


if __name__ == "__main__":
    main()
