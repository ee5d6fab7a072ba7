"""ctypes front-end of the CPU oracle (``liboracle.so``) and of the reference shims (``_ref/``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the CPU-baseline leg of
the benchmark, never by the product package.  Each wrapper is a one-to-one call of the C function
of the same name in ``cphnsw_oracle.cpp`` / ``ref_shim.cpp``; see those files for the reference
file:line every function follows.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
INVALID = 0xFFFFFFFF
FHT_SCALAR, FHT_AVX2, FHT_AVX512 = 0, 1, 2


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def next_pow2(n):
    p = 1
    while p < n:
        p *= 2
    return p


def _comp_dtype(comp_bytes):
    return np.uint8 if comp_bytes == 1 else np.uint16


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            raise RuntimeError("oracle/liboracle.so missing: run `make -C oracle`")
        _lib = C.CDLL(path)
    return _lib


def use_tuned_build():
    """Switches this module to the tuned build of the same source (`make -C oracle native`: -O3 -march=native,
    AVX-512 gather score and byte compare where the host has them, sorted-array beam) - the benchmark's CPU
    baseline.  Built on the host it runs on; returns False (and keeps the plain build) when that fails."""
    global _lib
    import subprocess
    path = os.path.join(_HERE, "_native", "liboracle_tuned.so")
    try:
        subprocess.run(["make", "-C", _HERE, "native"], check=True, capture_output=True, timeout=300)
        tuned = C.CDLL(path)
        if tuned.orc_is_tuned() != 1:
            return False
    except Exception:
        return False
    _lib = tuned
    return True


def use_plain_build():
    global _lib
    _lib = None
    lib()


def is_tuned():
    return bool(lib().orc_is_tuned())


def num_threads():
    return lib().orc_num_threads()


def sign_tables(dim, K, seed=42):
    P = next_pow2(dim)
    out = np.empty((K, 3, P), np.int8)
    lib().orc_sign_tables(C.c_uint64(dim), C.c_uint64(K), C.c_uint64(seed), _ptr(out))
    return out


def fht(v, convention=FHT_SCALAR):
    v = np.ascontiguousarray(v, np.float32).copy()
    lib().orc_fht(_ptr(v), C.c_uint64(v.size), C.c_int(convention))
    return v


def encode(x, K, comp_bytes, signs, convention=FHT_AVX512, want_rotated=False):
    x = np.ascontiguousarray(x, np.float32)
    n, dim = x.shape
    P = next_pow2(dim)
    signs = np.ascontiguousarray(signs, np.int8)
    assert signs.shape == (K, 3, P)
    codes = np.empty((n, K), _comp_dtype(comp_bytes))
    rot = np.empty((n, K, P), np.float32) if want_rotated else None
    mag = np.empty((n, K), np.float32) if want_rotated else None
    lib().orc_encode(_ptr(x), C.c_uint64(n), C.c_uint64(dim), C.c_uint64(K), C.c_uint64(comp_bytes),
                     _ptr(signs), C.c_int(convention), _ptr(codes), _ptr(rot), _ptr(mag))
    return (codes, rot, mag) if want_rotated else codes


class residual_weighting:
    """Context manager: inside it every code distance of the oracle is the combined distance of
    residual codes, (h_primary << shift) + h_residual, the first `primary` components being primary."""

    def __init__(self, primary, shift):
        self.primary, self.shift = primary, shift

    def __enter__(self):
        lib().orc_set_residual_weighting(C.c_uint64(self.primary), C.c_uint32(self.shift))
        return self

    def __exit__(self, *exc):
        lib().orc_set_residual_weighting(C.c_uint64(0), C.c_uint32(0))
        return False


def code_distance(a, b):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert a.dtype == b.dtype and a.shape[1] == b.shape[1]
    out = np.empty((a.shape[0], b.shape[0]), np.uint16)
    lib().orc_code_distance(_ptr(a), C.c_uint64(a.shape[0]), _ptr(b), C.c_uint64(b.shape[0]),
                            C.c_uint64(a.shape[1]), C.c_uint64(a.dtype.itemsize), _ptr(out))
    return out


def knn_graph(codes, k, row_begin=0, row_end=None):
    codes = np.ascontiguousarray(codes)
    n, K = codes.shape
    row_end = n if row_end is None else row_end
    nb = np.empty((row_end - row_begin, k), np.uint32)
    ds = np.empty((row_end - row_begin, k), np.uint16)
    lib().orc_knn_graph(_ptr(codes), C.c_uint64(n), C.c_uint64(K), C.c_uint64(codes.dtype.itemsize),
                        C.c_uint64(k), C.c_uint64(row_begin), C.c_uint64(row_end), _ptr(nb), _ptr(ds))
    return nb, ds


def select_neighbors(codes, cand, M, keep_pruned=True, row_begin=0):
    codes = np.ascontiguousarray(codes)
    cand = np.ascontiguousarray(cand, np.uint32)
    n, K = codes.shape
    rows, k = cand.shape
    adj = np.empty((rows, M), np.uint32)
    lib().orc_select_neighbors(_ptr(codes), C.c_uint64(n), C.c_uint64(K), C.c_uint64(codes.dtype.itemsize),
                               _ptr(cand), C.c_uint64(k), C.c_uint64(M), C.c_int(int(keep_pruned)),
                               C.c_uint64(row_begin), C.c_uint64(row_begin + rows), _ptr(adj))
    return adj


def rank_prune(cand, M, alpha=1.1):
    """Rank-based (CAGRA) pruning of the kNN lists of all nodes: cand [n][k] -> adjacency [n][M]."""
    cand = np.ascontiguousarray(cand, np.uint32)
    n, k = cand.shape
    adj = np.empty((n, M), np.uint32)
    lib().orc_rank_prune(_ptr(cand), C.c_uint64(n), C.c_uint64(k), C.c_uint64(M), C.c_float(alpha), _ptr(adj))
    return adj


def exact_candidates(base, k, row_begin=0, row_end=None):
    """Exact nearest neighbours by -<x,y> of rows [row_begin, row_end) among all rows, the row itself removed."""
    base = np.ascontiguousarray(base, np.float32)
    n, dim = base.shape
    row_end = n if row_end is None else row_end
    cand = np.empty((row_end - row_begin, k), np.uint32)
    lib().orc_exact_candidates(_ptr(base), C.c_uint64(n), C.c_uint64(dim), C.c_uint64(k), C.c_uint64(row_begin),
                               C.c_uint64(row_end), _ptr(cand))
    return cand


def select_neighbors_exact(base, cand, M, keep_pruned=True, row_begin=0):
    """select_neighbors on exact fp32 distances (the legacy hybrid construction)."""
    base = np.ascontiguousarray(base, np.float32)
    cand = np.ascontiguousarray(cand, np.uint32)
    n, dim = base.shape
    rows, k = cand.shape
    adj = np.empty((rows, M), np.uint32)
    lib().orc_select_neighbors_exact(_ptr(base), C.c_uint64(n), C.c_uint64(dim), _ptr(cand), C.c_uint64(k), C.c_uint64(M),
                                     C.c_int(int(keep_pruned)), C.c_uint64(row_begin), C.c_uint64(row_begin + rows), _ptr(adj))
    return adj


def set_threads(threads):
    """Sets the OpenMP thread count of the oracle (returns the count now in force)."""
    return int(lib().orc_set_threads(C.c_int(int(threads))))


def search(tables, codes, adj, entry_ids, ef, k, want_stats=False, n_seed=None):
    """n_seed: how many of the scored entry ids seed the walk (None = all of them)."""
    tables = np.ascontiguousarray(tables, np.float32)
    codes = np.ascontiguousarray(codes)
    adj = np.ascontiguousarray(adj, np.uint32)
    entry_ids = np.ascontiguousarray(entry_ids, np.uint32)
    nq, K, P = tables.shape
    n, M = adj.shape
    ids = np.empty((nq, k), np.uint32)
    dist = np.empty((nq, k), np.float32)
    stats = np.zeros((nq, 2), np.uint32)
    lib().orc_search(_ptr(tables), C.c_uint64(nq), C.c_uint64(K), C.c_uint64(P), _ptr(codes),
                     C.c_uint64(codes.dtype.itemsize), C.c_uint64(n), _ptr(adj), C.c_uint64(M),
                     _ptr(entry_ids), C.c_uint64(entry_ids.size),
                     C.c_uint64(entry_ids.size if n_seed is None else n_seed), C.c_uint64(ef), C.c_uint64(k),
                     _ptr(ids), _ptr(dist), _ptr(stats))
    return (ids, dist, stats) if want_stats else (ids, dist)


def search_codes(qcodes, codes, adj, entry_ids, ef, k, n_seed=None):
    """The walk under the symmetric code distance to qcodes[q] (distances returned as floats)."""
    qcodes = np.ascontiguousarray(qcodes)
    codes = np.ascontiguousarray(codes)
    adj = np.ascontiguousarray(adj, np.uint32)
    entry_ids = np.ascontiguousarray(entry_ids, np.uint32)
    nq, K = qcodes.shape
    n, M = adj.shape
    ids = np.empty((nq, k), np.uint32)
    dist = np.empty((nq, k), np.float32)
    lib().orc_search_codes(_ptr(qcodes), C.c_uint64(nq), C.c_uint64(K), _ptr(codes), C.c_uint64(codes.dtype.itemsize),
                           C.c_uint64(n), _ptr(adj), C.c_uint64(M), _ptr(entry_ids), C.c_uint64(entry_ids.size),
                           C.c_uint64(entry_ids.size if n_seed is None else n_seed), C.c_uint64(ef), C.c_uint64(k),
                           _ptr(ids), _ptr(dist), None)
    return ids, dist


def probe_codes(rotated, comp_bytes, T):
    """Multiprobe sequence: [nq][T][K] probe codes, the primary code first."""
    rotated = np.ascontiguousarray(rotated, np.float32)
    nq, K, P = rotated.shape
    out = np.empty((nq, T, K), _comp_dtype(comp_bytes))
    lib().orc_probe_codes(_ptr(rotated), C.c_uint64(nq), C.c_uint64(K), C.c_uint64(P), C.c_uint64(comp_bytes),
                          C.c_uint64(T), _ptr(out))
    return out


def search_multiprobe(rotated, comp_bytes, codes, adj, entry_ids, ef, k, T, n_seed=None):
    """search_multiprobe(q, k, ef, num_probes): one symmetric-distance walk per probe code, merged."""
    pc = probe_codes(rotated, comp_bytes, T)
    nq, _, K = pc.shape
    ids, dist = search_codes(pc.reshape(nq * T, K), codes, adj, entry_ids, ef, k, n_seed)
    oi = np.empty((nq, k), np.uint32)
    od = np.empty((nq, k), np.float32)
    lib().orc_merge_probes(_ptr(ids), _ptr(dist), C.c_uint64(nq), C.c_uint64(T), C.c_uint64(k), _ptr(oi), _ptr(od))
    return oi, od


def rerank(queries, base, cand, k):
    queries = np.ascontiguousarray(queries, np.float32)
    base = np.ascontiguousarray(base, np.float32)
    cand = np.ascontiguousarray(cand, np.uint32)
    nq, dim = queries.shape
    ids = np.empty((nq, k), np.uint32)
    dist = np.empty((nq, k), np.float32)
    lib().orc_rerank(_ptr(queries), C.c_uint64(nq), C.c_uint64(dim), _ptr(base), _ptr(cand),
                     C.c_uint64(cand.shape[1]), C.c_uint64(k), _ptr(ids), _ptr(dist))
    return ids, dist


def ground_truth(queries, base, k, want_dist=False):
    queries = np.ascontiguousarray(queries, np.float32)
    base = np.ascontiguousarray(base, np.float32)
    ids = np.empty((queries.shape[0], k), np.uint32)
    dist = np.empty((queries.shape[0], k), np.float32) if want_dist else None
    lib().orc_ground_truth(_ptr(queries), C.c_uint64(queries.shape[0]), _ptr(base),
                           C.c_uint64(base.shape[0]), C.c_uint64(base.shape[1]), C.c_uint64(k), _ptr(ids),
                           _ptr(dist) if want_dist else None)
    return (ids, dist) if want_dist else ids


def brute_force(rotated, codes, k):
    """Exhaustive top-k by asymmetric CP score; rotated is float32 [nq][K][P]."""
    rotated = np.ascontiguousarray(rotated, np.float32)
    nq, K, P = rotated.shape
    codes = np.ascontiguousarray(codes)
    ids = np.empty((nq, k), np.uint32)
    dist = np.empty((nq, k), np.float32)
    lib().orc_brute_force(_ptr(rotated), C.c_uint64(nq), C.c_uint64(K), C.c_uint64(P), _ptr(codes),
                          C.c_uint64(codes.dtype.itemsize), C.c_uint64(codes.shape[0]), C.c_uint64(k), _ptr(ids), _ptr(dist))
    return ids, dist


def calibration_pairs(n, num_samples, seed):
    u = np.empty(num_samples, np.uint32)
    v = np.empty(num_samples, np.uint32)
    lib().orc_calibration_pairs(C.c_uint64(n), C.c_uint64(num_samples), C.c_uint64(seed), _ptr(u), _ptr(v))
    return u, v


def linear_fit(x, y):
    x = np.ascontiguousarray(x, np.float32)
    y = np.ascontiguousarray(y, np.float32)
    out = np.empty(3, np.float64)
    lib().orc_linear_fit(_ptr(x), _ptr(y), C.c_uint64(x.size), _ptr(out))
    return float(out[0]), float(out[1]), float(out[2])


def calibrate(base, codes, signs, K, comp_bytes, convention, num_samples, seed):
    """(alpha, beta, r_squared, x, y) of the legacy index's calibrate(num_samples, seed)."""
    base = np.ascontiguousarray(base, np.float32)
    codes = np.ascontiguousarray(codes)
    n, dim = base.shape
    u, v = calibration_pairs(n, num_samples, seed)
    _, rot, _ = encode(base[u], K, comp_bytes, signs, convention, want_rotated=True)
    x = np.empty(num_samples, np.float32)
    y = np.empty(num_samples, np.float32)
    lib().orc_calibration_samples(_ptr(rot), C.c_uint64(K), C.c_uint64(rot.shape[2]), _ptr(codes),
                                  C.c_uint64(codes.dtype.itemsize), _ptr(base), C.c_uint64(n), C.c_uint64(dim),
                                  C.c_uint64(num_samples), _ptr(u), _ptr(v), _ptr(x), _ptr(y))
    return linear_fit(x, y) + (x, y)


def connectivity(adj, entry_ids):
    adj = np.ascontiguousarray(adj, np.uint32)
    entry_ids = np.ascontiguousarray(entry_ids, np.uint32)
    f = lib().orc_connectivity
    f.restype = C.c_uint64
    return int(f(_ptr(adj), C.c_uint64(adj.shape[0]), C.c_uint64(adj.shape[1]), _ptr(entry_ids), C.c_uint64(entry_ids.size)))


def recall_at_k(found, truth, k):
    """|retrieved ∩ truth| / k averaged over queries (evaluation/metrics/recall.hpp:22-39)."""
    hits = 0
    for f, t in zip(found[:, :k], truth[:, :k]):
        hits += len(set(f.tolist()) & set(t.tolist()))
    return hits / (truth.shape[0] * k)


# ---------------------------------------------------------------------------------------------
# reference shims (present only where the reference checkout was available at build time)

_CONV_NAME = {FHT_SCALAR: "scalar", FHT_AVX2: "avx2", FHT_AVX512: "avx512"}


def _cpu_has(flag):
    try:
        with open("/proc/cpuinfo") as f:
            return flag in f.read().split("flags", 1)[1].split("\n", 1)[0].split()
    except Exception:
        return False


def ref_available(convention):
    path = os.path.join(_HERE, "_ref", "libcphnsw_ref_%s.so" % _CONV_NAME[convention])
    if not os.path.exists(path):
        return False
    need = {FHT_SCALAR: None, FHT_AVX2: "avx2", FHT_AVX512: "avx512f"}[convention]
    return need is None or _cpu_has(need)


class Ref:
    """The reference's own headers compiled with the ISA flags of one convention."""

    def __init__(self, convention):
        if not ref_available(convention):
            raise RuntimeError("reference shim for convention %d not available" % convention)
        self.l = C.CDLL(os.path.join(_HERE, "_ref", "libcphnsw_ref_%s.so" % _CONV_NAME[convention]))
        assert self.l.ref_convention() == convention

    def fht(self, v):
        v = np.ascontiguousarray(v, np.float32).copy()
        self.l.ref_fht(_ptr(v), C.c_uint64(v.size))
        return v

    def fht_scalar(self, v):
        v = np.ascontiguousarray(v, np.float32).copy()
        self.l.ref_fht_scalar(_ptr(v), C.c_uint64(v.size))
        return v

    def sign_tables(self, dim, K, seed=42):
        out = np.empty((K, 3, next_pow2(dim)), np.int8)
        self.l.ref_sign_tables(C.c_uint64(dim), C.c_uint64(K), C.c_uint64(seed), _ptr(out))
        return out

    def argmax_abs(self, v):
        v = np.ascontiguousarray(v, np.float32)
        idx = C.c_uint64()
        mag = C.c_float()
        self.l.ref_argmax_abs(_ptr(v), C.c_uint64(v.size), C.byref(idx), C.byref(mag))
        return idx.value, mag.value

    def encode(self, x, K, comp_bytes, seed=42, want_rotated=False):
        x = np.ascontiguousarray(x, np.float32)
        n, dim = x.shape
        P = next_pow2(dim)
        codes = np.empty((n, K), _comp_dtype(comp_bytes))
        rot = np.empty((n, K, P), np.float32) if want_rotated else None
        mag = np.empty((n, K), np.float32) if want_rotated else None
        self.l.ref_encode(_ptr(x), C.c_uint64(n), C.c_uint64(dim), C.c_uint64(K), C.c_uint64(comp_bytes),
                          C.c_uint64(seed), _ptr(codes), _ptr(rot), _ptr(mag))
        return (codes, rot, mag) if want_rotated else codes

    def encode_batch_signbits64(self, x, seed=42):
        """The unified encoder CPEncoder<64,0>: one uint64 of sign bits per vector."""
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[0], np.uint64)
        self.l.ref_encode_batch_signbits64(_ptr(x), C.c_uint64(x.shape[0]), C.c_uint64(x.shape[1]), C.c_uint64(seed), _ptr(out))
        return out

    def encode_batch_residual_32_16(self, x, seed=42):
        """The unified encoder CPEncoder<32,16>: (primary uint64 word, residual uint64 word) per vector."""
        x = np.ascontiguousarray(x, np.float32)
        prim = np.empty(x.shape[0], np.uint64)
        res = np.empty(x.shape[0], np.uint64)
        self.l.ref_encode_batch_residual_32_16(_ptr(x), C.c_uint64(x.shape[0]), C.c_uint64(x.shape[1]), C.c_uint64(seed),
                                               _ptr(prim), _ptr(res))
        return prim, res

    def hamming_combined_32_16_s2(self, pa, ra, pb, rb):
        """The reference's hamming_combined_scalar<32,16,2> between codes given as (primary, residual) words."""
        pa, ra, pb, rb = (np.ascontiguousarray(v, np.uint64) for v in (pa, ra, pb, rb))
        out = np.empty((pa.size, pb.size), np.uint32)
        self.l.ref_hamming_combined_32_16_s2(_ptr(pa), _ptr(ra), C.c_uint64(pa.size), _ptr(pb), _ptr(rb), C.c_uint64(pb.size),
                                             _ptr(out))
        return out

    def hamming64(self, a, b):
        """The reference's hamming_primary_scalar<64> between packed codes (scalar build only)."""
        a = np.ascontiguousarray(a, np.uint64)
        b = np.ascontiguousarray(b, np.uint64)
        out = np.empty((a.size, b.size), np.uint32)
        self.l.ref_hamming64(_ptr(a), C.c_uint64(a.size), _ptr(b), C.c_uint64(b.size), _ptr(out))
        return out

    def encode_batch_signbits32(self, x, seed=42):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape[0], np.uint32)
        self.l.ref_encode_batch_signbits32(_ptr(x), C.c_uint64(x.shape[0]), C.c_uint64(x.shape[1]),
                                           C.c_uint64(seed), _ptr(out))
        return out


def ref_search_available():
    return os.path.exists(os.path.join(_HERE, "_ref", "libcphnsw_ref_search.so"))


class RefSearch:
    """The reference's own graph walk (include/cphnsw/search/search_engine.hpp:86-193), built by
    `make -C oracle ref` from a throw-away patched copy of its headers (see ref_search_shim.cpp).
    Codes are packed sign bits; every call returns W in full (k = ef), ascending by distance."""

    def __init__(self):
        self.l = C.CDLL(os.path.join(_HERE, "_ref", "libcphnsw_ref_search.so"))

    def _out(self, nq, ef):
        return np.empty((nq, ef), np.uint32), np.empty((nq, ef), np.float32), np.empty(nq, np.uint32)

    def search_64(self, codes, adj, qcodes, entry, ef):
        codes = np.ascontiguousarray(codes, np.uint64)
        qcodes = np.ascontiguousarray(qcodes, np.uint64)
        adj = np.ascontiguousarray(adj, np.uint32)
        entry = np.ascontiguousarray(entry, np.uint32)
        ids, dist, cnt = self._out(qcodes.shape[0], ef)
        self.l.ref_search_64(_ptr(codes), C.c_uint64(codes.shape[0]), _ptr(adj), C.c_uint64(adj.shape[1]), _ptr(qcodes),
                             C.c_uint64(qcodes.shape[0]), _ptr(entry), C.c_uint64(entry.size), C.c_uint64(ef),
                             _ptr(ids), _ptr(dist), _ptr(cnt))
        return ids, dist, cnt

    def search_32_16_s2(self, primary, residual, adj, q_primary, q_residual, entry, ef):
        arrs = [np.ascontiguousarray(a, np.uint64) for a in (primary, residual, q_primary, q_residual)]
        adj = np.ascontiguousarray(adj, np.uint32)
        entry = np.ascontiguousarray(entry, np.uint32)
        ids, dist, cnt = self._out(arrs[2].shape[0], ef)
        self.l.ref_search_32_16_s2(_ptr(arrs[0]), _ptr(arrs[1]), C.c_uint64(arrs[0].shape[0]), _ptr(adj),
                                   C.c_uint64(adj.shape[1]), _ptr(arrs[2]), _ptr(arrs[3]), C.c_uint64(arrs[2].shape[0]),
                                   _ptr(entry), C.c_uint64(entry.size), C.c_uint64(ef), _ptr(ids), _ptr(dist), _ptr(cnt))
        return ids, dist, cnt


def pack_sign_bits(codes):
    """One-byte sign components [n][K <= 64] -> uint64[n], bit r = component r (core/codes.hpp:21-52)."""
    codes = np.asarray(codes)
    return ((codes.astype(np.uint64) & np.uint64(1)) << np.arange(codes.shape[1], dtype=np.uint64)).sum(axis=1).astype(np.uint64)


def unpack_sign_bits(words, K):
    words = np.asarray(words, np.uint64)
    return ((words[:, None] >> np.arange(K, dtype=np.uint64)) & np.uint64(1)).astype(np.uint8)
