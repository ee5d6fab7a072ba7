"""The oracle's beam search against the reference's own walk, SearchEngine<Policy>::search
(include/cphnsw/search/search_engine.hpp:86-193), recorded in tests/golden/walk_golden.npz by
tests/golden/make_walk_golden.py (and re-run live where oracle/_ref holds the reference build).

The reference orders candidates on `distance` alone; the oracle (and the library) on (distance, id).
On the tie-free cases the two orders coincide and the walks must agree exactly: same members of W,
same order, same distances - that pins the control flow (seeding, visited marks, admission rule,
termination, extraction).  Where distances tie, which of several equal candidates a heap keeps is
an accident of the heap, later expansions differ, and only aggregate agreement can be asked for.
Declared deviation: the reference seeds W with every entry point even beyond ef
(search_engine.hpp:105-115); the oracle bounds W at ef from the start, so cases keep n_entry <= ef.
"""
import os

import numpy as np
import pytest

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "walk_golden.npz"))
INVALID = 0xFFFFFFFF


def _entries(row):
    return row[row != INVALID]


@pytest.mark.parametrize("c", range(GOLD["tf64_q"].shape[0]))
def test_tie_free_walk_equals_reference_64(oracle, c):
    ef = int(GOLD["tf64_ef"][c])
    codes = oracle.unpack_sign_bits(GOLD["tf64_codes"][c], 64)
    q = oracle.unpack_sign_bits(GOLD["tf64_q"][c:c + 1], 64)
    ids, dist = oracle.search_codes(q, codes, GOLD["tf64_adj"][c], _entries(GOLD["tf64_entry"][c]), ef, ef)
    assert np.array_equal(ids[0], GOLD["tf64_ids"][c, :ef])
    assert np.array_equal(dist[0], GOLD["tf64_dist"][c, :ef])
    assert int((ids[0] != INVALID).sum()) == int(GOLD["tf64_count"][c])


@pytest.mark.parametrize("c", range(GOLD["tfr_qp"].shape[0]))
def test_tie_free_walk_equals_reference_residual(oracle, c):
    # CPHNSWIndex<32, 16, 2>: one-byte sign components, 32 primary then 16 residual, distance (h_p << 2) + h_r
    ef = int(GOLD["tfr_ef"][c])
    codes = np.concatenate([oracle.unpack_sign_bits(GOLD["tfr_prim"][c], 32), oracle.unpack_sign_bits(GOLD["tfr_resi"][c], 16)], axis=1)
    q = np.concatenate([oracle.unpack_sign_bits(GOLD["tfr_qp"][c:c + 1], 32), oracle.unpack_sign_bits(GOLD["tfr_qr"][c:c + 1], 16)], axis=1)
    with oracle.residual_weighting(32, 2):
        ids, dist = oracle.search_codes(q, codes, GOLD["tfr_adj"][c], _entries(GOLD["tfr_entry"][c]), ef, ef)
    assert np.array_equal(ids[0], GOLD["tfr_ids"][c, :ef])
    assert np.array_equal(dist[0], GOLD["tfr_dist"][c, :ef])
    assert int((ids[0] != INVALID).sum()) == int(GOLD["tfr_count"][c])


def test_walk_with_ties_agrees_in_aggregate(oracle):
    # 64-bit Hamming distances tie massively; the two tie rules then explore different nodes, so W may
    # differ even below the worst distance.  What must hold: the same quality of result.
    ef = int(GOLD["tie_ef"])
    codes = oracle.unpack_sign_bits(GOLD["tie_codes"], 64)
    q = oracle.unpack_sign_bits(GOLD["tie_q"], 64)
    ids, dist = oracle.search_codes(q, codes, GOLD["tie_adj"], GOLD["tie_entry"], ef, ef)
    rd = GOLD["tie_dist"]
    assert abs(float(dist.mean()) - float(rd.mean())) < 0.05
    assert float(np.mean(dist[:, 0] == rd[:, 0])) == 1.0  # the nearest distance found is the same
    same_best10 = np.mean([np.array_equal(np.sort(a[:10]), np.sort(b[:10])) for a, b in zip(dist, rd)])
    assert same_best10 >= 0.95


def test_reference_walk_live(oracle):
    """Where the reference build is present, the fixture is what it returns now."""
    if not oracle.ref_search_available():
        pytest.skip("oracle/_ref/libcphnsw_ref_search.so not built (no reference checkout)")
    R = oracle.RefSearch()
    for c in range(0, GOLD["tf64_q"].shape[0], 5):
        ef = int(GOLD["tf64_ef"][c])
        ids, dist, cnt = R.search_64(GOLD["tf64_codes"][c], GOLD["tf64_adj"][c], GOLD["tf64_q"][c:c + 1],
                                     _entries(GOLD["tf64_entry"][c]), ef)
        assert np.array_equal(ids[0], GOLD["tf64_ids"][c, :ef]) and cnt[0] == GOLD["tf64_count"][c]
