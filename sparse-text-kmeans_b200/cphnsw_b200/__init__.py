"""ctypes binding of ``libcphnsw_b200.so`` (C ABI in ``include/cphnsw_b200.h``).

``CPHNSWIndex`` mirrors the legacy ``CPHNSWIndex<ComponentT,K>`` surface of the reference (use sites:
evaluation/eval_sift.cpp:228-266,387, evaluation/eval_master.cpp:89,145, evaluation/eval_main.cpp:43):
``add_batch`` / ``add_batch_parallel`` / ``search`` / ``search_and_rerank`` with host (numpy) arrays in
and out, plus batched forms and the individual stages (``encode``, ``code_distance``, ``knn_graph``,
``select_neighbors``).  Errors that the reference raises as ``std::invalid_argument`` surface as
``ValueError``; everything else as ``CPHNSWError``.

There is no CPU implementation behind this module: importing it without the built library, or
constructing an index without a B200, raises.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libcphnsw_b200.so")

INVALID_NODE = 0xFFFFFFFF
FHT_SCALAR, FHT_AVX2, FHT_AVX512 = 0, 1, 2
E_INVALID, E_CUDA, E_STATE, E_UNSUPPORTED, E_DEVICE_WAIT = -1, -2, -3, -4, -5

# every symbol include/cphnsw_b200.h declares
EXPORTS = [
    "cphnsw_b200_last_error", "cphnsw_b200_device_count", "cphnsw_b200_create", "cphnsw_b200_destroy",
    "cphnsw_b200_set_param", "cphnsw_b200_get_param", "cphnsw_b200_dim", "cphnsw_b200_padded_dim",
    "cphnsw_b200_size", "cphnsw_b200_get_sign_tables", "cphnsw_b200_set_sign_tables", "cphnsw_b200_encode",
    "cphnsw_b200_encode_queries", "cphnsw_b200_code_distance", "cphnsw_b200_knn_graph",
    "cphnsw_b200_select_neighbors", "cphnsw_b200_add_batch_parallel", "cphnsw_b200_get_codes",
    "cphnsw_b200_get_adjacency", "cphnsw_b200_get_entry_ids", "cphnsw_b200_search_batch",
    "cphnsw_b200_search_and_rerank_batch", "cphnsw_b200_encode_dev", "cphnsw_b200_code_distance_dev",
    "cphnsw_b200_knn_graph_dev", "cphnsw_b200_select_neighbors_dev", "cphnsw_b200_install_dev",
    "cphnsw_b200_search_dev", "cphnsw_b200_check_device_status", "cphnsw_b200_launch_count",
    "cphnsw_b200_kernel_time", "cphnsw_b200_code_distance_noalloc", "cphnsw_b200_search_multiprobe_batch",
    "cphnsw_b200_probe_codes", "cphnsw_b200_brute_force_search_batch", "cphnsw_b200_verify_connectivity",
    "cphnsw_b200_calibrate", "cphnsw_b200_get_calibration", "cphnsw_b200_search_calibrated_batch",
    "cphnsw_b200_save", "cphnsw_b200_load", "cphnsw_b200_add_batch", "cphnsw_b200_get_binary_codes",
    "cphnsw_b200_create_binary", "cphnsw_b200_set_exact_base", "cphnsw_b200_exact_search_batch",
    "cphnsw_b200_rerank_batch", "cphnsw_b200_exact_search_dev", "cphnsw_b200_rank_prune",
    "cphnsw_b200_rank_reorder_dev", "cphnsw_b200_rank_merge_dev", "cphnsw_b200_install",
    "cphnsw_b200_search_codes_batch", "cphnsw_b200_get_code", "cphnsw_b200_sharded_create", "cphnsw_b200_sharded_load",
    "cphnsw_b200_sharded_destroy", "cphnsw_b200_sharded_gpus", "cphnsw_b200_sharded_size", "cphnsw_b200_sharded_replica",
    "cphnsw_b200_sharded_set_param", "cphnsw_b200_sharded_add_batch_parallel", "cphnsw_b200_sharded_add_batch",
    "cphnsw_b200_sharded_search", "cphnsw_b200_sharded_stage_times",
]


class CPHNSWError(RuntimeError):
    pass


_lib = None


def load_library():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CPHNSWError("%s not found: run `python sparse-text-kmeans_b200/build.py`" % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        lib.cphnsw_b200_last_error.restype = C.c_char_p
        for name in ("cphnsw_b200_dim", "cphnsw_b200_padded_dim", "cphnsw_b200_size", "cphnsw_b200_launch_count",
                     "cphnsw_b200_sharded_size"):
            getattr(lib, name).restype = C.c_uint64
            getattr(lib, name).argtypes = [C.c_void_p]
        lib.cphnsw_b200_sharded_replica.restype = C.c_void_p
        lib.cphnsw_b200_sharded_replica.argtypes = [C.c_void_p, C.c_int]
        _lib = lib
    return _lib


def device_count():
    return load_library().cphnsw_b200_device_count()


def _check(rc):
    if rc == 0:
        return
    msg = load_library().cphnsw_b200_last_error().decode()
    if rc == E_INVALID:
        raise ValueError(msg)
    raise CPHNSWError("[%d] %s" % (rc, msg))


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u64(v):
    return C.c_uint64(int(v))


def _u32(v):
    return C.c_uint32(int(v))


def code_distance_noalloc(d_a, na, d_b, nb, K, component_bytes, d_out, stream=0):
    """Allocation-free code distance on the current CUDA device (raw device addresses in and out).

    For hosts that may not allocate device memory once running; inputs are limited to what fits the
    library's built-in 1 MiB scratch (see ``cphnsw_b200_code_distance_noalloc`` in the C header).
    """
    _check(load_library().cphnsw_b200_code_distance_noalloc(
        C.c_void_p(d_a), _u64(na), C.c_void_p(d_b), _u64(nb), _u32(K), _u32(component_bytes), C.c_void_p(d_out),
        C.c_void_p(stream)))


class CPHNSWIndex:
    """Drop-in mirror of ``CPHNSWIndex<ComponentT,K>``; ``component_bytes`` selects ComponentT."""

    def __init__(self, dim, M=32, ef_construction=200, K=32, component_bytes=1, seed=42,
                 fht_convention=FHT_AVX512, device=0):
        self._lib = load_library()
        self._h = C.c_void_p()
        _check(self._lib.cphnsw_b200_create(_u64(dim), _u32(K), _u32(component_bytes), _u32(M), _u32(ef_construction),
                                            _u64(seed), C.c_int(fht_convention), C.c_int(device), C.byref(self._h)))
        self.dim, self.K, self.M, self.component_bytes = dim, K, M, component_bytes
        self.padded_dim = int(self._lib.cphnsw_b200_padded_dim(self._h))
        self.code_dtype = np.uint8 if component_bytes == 1 else np.uint16

    @classmethod
    def binary(cls, dim, M=32, ef_construction=200, K=64, seed=42, fht_convention=FHT_AVX512, device=0):
        """The unified index's binary-code variant: K sign bits per vector, Hamming metric (one-byte
        components whatever the dimension)."""
        self = cls.__new__(cls)
        self._lib = load_library()
        self._h = C.c_void_p()
        _check(self._lib.cphnsw_b200_create_binary(_u64(dim), _u32(K), _u32(M), _u32(ef_construction), _u64(seed),
                                                   C.c_int(fht_convention), C.c_int(device), C.byref(self._h)))
        self.dim, self.K, self.M, self.component_bytes = dim, K, M, 1
        self.padded_dim = int(self._lib.cphnsw_b200_padded_dim(self._h))
        self.code_dtype = np.uint8
        return self

    def save(self, path):
        """Writes the whole index (parameters, sign tables, vectors, codes, adjacency) to one file."""
        _check(self._lib.cphnsw_b200_save(self._h, os.fsencode(path)))

    @classmethod
    def load(cls, path, device=0):
        """A new index holding exactly what ``save`` wrote; nothing is re-encoded or rebuilt."""
        self = cls.__new__(cls)
        self._lib = load_library()
        self._h = C.c_void_p()
        _check(self._lib.cphnsw_b200_load(os.fsencode(path), C.c_int(device), C.byref(self._h)))
        self.dim = int(self._lib.cphnsw_b200_dim(self._h))
        self.K, self.M, self.component_bytes = (int(self.get_param(n)) for n in ("K", "M", "component_bytes"))
        self.padded_dim = int(self._lib.cphnsw_b200_padded_dim(self._h))
        self.code_dtype = np.uint8 if self.component_bytes == 1 else np.uint16
        return self

    def close(self):
        h = getattr(self, "_h", None)
        if h is not None and h.value:
            if not getattr(self, "_borrowed", False):  # a replica of a ShardedIndex belongs to it
                self._lib.cphnsw_b200_destroy(h)
            h.value = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown: module globals may already be gone
            pass

    @property
    def handle(self):
        return self._h

    # ---- parameters -------------------------------------------------------------------------
    def set_param(self, name, value):
        _check(self._lib.cphnsw_b200_set_param(self._h, name.encode(), C.c_double(value)))

    def get_param(self, name):
        v = C.c_double()
        _check(self._lib.cphnsw_b200_get_param(self._h, name.encode(), C.byref(v)))
        return v.value

    def size(self):
        return int(self._lib.cphnsw_b200_size(self._h))

    def launch_count(self):
        return int(self._lib.cphnsw_b200_launch_count(self._h))

    def sign_tables(self):
        out = np.empty((self.K, 3, self.padded_dim), np.int8)
        _check(self._lib.cphnsw_b200_get_sign_tables(self._h, _p(out)))
        return out

    def set_sign_tables(self, signs):
        signs = np.ascontiguousarray(signs, np.int8)
        if signs.shape != (self.K, 3, self.padded_dim):
            raise ValueError("sign tables must be int8[K][3][padded_dim]")
        _check(self._lib.cphnsw_b200_set_sign_tables(self._h, _p(signs)))

    # ---- stages --------------------------------------------------------------------------------
    def _vecs(self, x):
        x = np.ascontiguousarray(x, np.float32)
        if x.ndim == 1:
            x = x[None, :]
        if x.ndim != 2 or x.shape[1] != self.dim:
            raise ValueError("expected float32[n][%d]" % self.dim)
        return x

    def _codes(self, c):
        c = np.ascontiguousarray(c, self.code_dtype)
        if c.ndim != 2 or c.shape[1] != self.K:
            raise ValueError("expected codes[n][%d]" % self.K)
        return c

    def encode(self, x):
        x = self._vecs(x)
        codes = np.empty((x.shape[0], self.K), self.code_dtype)
        _check(self._lib.cphnsw_b200_encode(self._h, _p(x), _u64(x.shape[0]), _p(codes)))
        return codes

    def encode_queries(self, q):
        """-> (codes [nq][K], rotated float32[nq][K][padded_dim], magnitudes float32[nq][K])."""
        q = self._vecs(q)
        nq = q.shape[0]
        codes = np.empty((nq, self.K), self.code_dtype)
        rot = np.empty((nq, self.K, self.padded_dim), np.float32)
        mag = np.empty((nq, self.K), np.float32)
        _check(self._lib.cphnsw_b200_encode_queries(self._h, _p(q), _u64(nq), _p(codes), _p(rot), _p(mag)))
        return codes, rot, mag

    def code_distance(self, a, b):
        a, b = self._codes(a), self._codes(b)
        out = np.empty((a.shape[0], b.shape[0]), np.uint16)
        _check(self._lib.cphnsw_b200_code_distance(self._h, _p(a), _u64(a.shape[0]), _p(b), _u64(b.shape[0]), _p(out)))
        return out

    def knn_graph(self, codes, k, row_begin=0, row_end=None):
        codes = self._codes(codes)
        n = codes.shape[0]
        row_end = n if row_end is None else row_end
        rows = max(0, row_end - row_begin)
        nbrs = np.empty((rows, k), np.uint32)
        dist = np.empty((rows, k), np.uint16)
        _check(self._lib.cphnsw_b200_knn_graph(self._h, _p(codes), _u64(n), _u32(k), _u64(row_begin), _u64(row_end),
                                               _p(nbrs), _p(dist)))
        return nbrs, dist

    def select_neighbors(self, codes, cand, M=None, keep_pruned=True, row_begin=0):
        codes = self._codes(codes)
        cand = np.ascontiguousarray(cand, np.uint32)
        M = self.M if M is None else M
        rows, k = cand.shape
        adj = np.empty((rows, M), np.uint32)
        _check(self._lib.cphnsw_b200_select_neighbors(self._h, _p(codes), _u64(codes.shape[0]), _p(cand), _u32(k),
                                                      _u64(row_begin), _u64(row_begin + rows), _u32(M),
                                                      C.c_int(int(keep_pruned)), _p(adj)))
        return adj

    # ---- index ---------------------------------------------------------------------------------
    def add_batch_parallel(self, x):
        x = self._vecs(x)
        _check(self._lib.cphnsw_b200_add_batch_parallel(self._h, _p(x), _u64(x.shape[0])))

    def add_batch(self, x):
        """Incremental insertion into the existing graph (bulk build on an empty index)."""
        x = self._vecs(x)
        _check(self._lib.cphnsw_b200_add_batch(self._h, _p(x), _u64(x.shape[0])))

    def add(self, vec):
        """Inserts one vector and returns its id (CPHNSWIndex::add, evaluation/eval_sift.cpp:239)."""
        nid = self.size()
        self.add_batch(self._vecs(vec))
        return nid

    def codes(self):
        out = np.empty((self.size(), self.K), self.code_dtype)
        _check(self._lib.cphnsw_b200_get_codes(self._h, _p(out)))
        return out

    def get_code(self, node_id):
        """CPHNSWIndex::get_code (evaluation/debug_code_storage.cpp:75): the K components of one node."""
        out = np.empty(self.K, self.code_dtype)
        _check(self._lib.cphnsw_b200_get_code(self._h, _u32(node_id), _p(out)))
        return out

    def install(self, vectors, codes, adj):
        """A complete index from host arrays: vectors [n][dim], codes [n][K], adjacency uint32 [n][M]."""
        vectors = self._vecs(vectors)
        codes = self._codes(codes)
        adj = np.ascontiguousarray(adj, np.uint32)
        assert codes.shape[0] == vectors.shape[0] == adj.shape[0] and adj.shape[1] == self.M
        _check(self._lib.cphnsw_b200_install(self._h, _p(vectors), _p(codes), _p(adj), _u64(vectors.shape[0])))

    def rank_prune(self, cand, M=None, alpha=1.1):
        """Rank-based (CAGRA) pruning of the kNN lists of ALL nodes: cand uint32 [n][k] -> adjacency [n][M]."""
        cand = np.ascontiguousarray(cand, np.uint32)
        M = self.M if M is None else M
        adj = np.empty((cand.shape[0], M), np.uint32)
        _check(self._lib.cphnsw_b200_rank_prune(self._h, _p(cand), _u64(cand.shape[0]), _u32(cand.shape[1]), _u32(M),
                                                C.c_float(alpha), _p(adj)))
        return adj

    def search_codes_batch(self, qcodes, k, ef, want_stats=False):
        """The walk under the symmetric code distance to the given query codes [nq][K]."""
        qcodes = self._codes(qcodes)
        nq = qcodes.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        stats = np.zeros((nq, 2), np.uint32) if want_stats else None
        _check(self._lib.cphnsw_b200_search_codes_batch(self._h, _p(qcodes), _u64(nq), _u32(k), _u32(ef), _p(ids), _p(dist),
                                                        _p(stats)))
        return (ids, dist, stats) if want_stats else (ids, dist)

    def binary_codes(self):
        """Sign bits of the stored codes, uint64 [size][(K+63)//64] (the unified index's primary code)."""
        out = np.zeros((self.size(), (self.K + 63) // 64), np.uint64)
        _check(self._lib.cphnsw_b200_get_binary_codes(self._h, _p(out)))
        return out

    def adjacency(self):
        out = np.empty((self.size(), self.M), np.uint32)
        _check(self._lib.cphnsw_b200_get_adjacency(self._h, _p(out)))
        return out

    def entry_ids(self):
        cnt = C.c_uint64()
        _check(self._lib.cphnsw_b200_get_entry_ids(self._h, None, C.byref(cnt)))
        out = np.empty(cnt.value, np.uint32)
        _check(self._lib.cphnsw_b200_get_entry_ids(self._h, _p(out), C.byref(cnt)))
        return out

    def search_batch(self, q, k, ef, want_stats=False):
        q = self._vecs(q)
        nq = q.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        stats = np.zeros((nq, 2), np.uint32) if want_stats else None
        _check(self._lib.cphnsw_b200_search_batch(self._h, _p(q), _u64(nq), _u32(k), _u32(ef), _p(ids), _p(dist), _p(stats)))
        return (ids, dist, stats) if want_stats else (ids, dist)

    def search_and_rerank_batch(self, q, k, ef, rerank_k, want_stats=False):
        q = self._vecs(q)
        nq = q.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        stats = np.zeros((nq, 2), np.uint32) if want_stats else None
        _check(self._lib.cphnsw_b200_search_and_rerank_batch(self._h, _p(q), _u64(nq), _u32(k), _u32(ef), _u32(rerank_k),
                                                             _p(ids), _p(dist), _p(stats)))
        return (ids, dist, stats) if want_stats else (ids, dist)

    def brute_force_search_batch(self, q, k):
        """The k nodes with the smallest asymmetric CP score among all stored nodes (no graph)."""
        q = self._vecs(q)
        nq = q.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        _check(self._lib.cphnsw_b200_brute_force_search_batch(self._h, _p(q), _u64(nq), _u32(k), _p(ids), _p(dist)))
        return ids, dist

    def brute_force_search(self, q, k):
        ids, dist = self.brute_force_search_batch(np.asarray(q, np.float32)[None, :], k)
        return [(int(i), float(d)) for i, d in zip(ids[0], dist[0]) if i != INVALID_NODE]

    def set_exact_base(self, base):
        """Vectors for exact_search / rerank to run over instead of the index's own (None drops them)."""
        if base is None:
            _check(self._lib.cphnsw_b200_set_exact_base(self._h, None, _u64(0)))
            return
        base = self._vecs(base)
        _check(self._lib.cphnsw_b200_set_exact_base(self._h, _p(base), _u64(base.shape[0])))

    def exact_search_batch(self, q, k):
        """Exact top-k by (-<q,x>, id) over the stored vectors (or the exact base): ground truth."""
        q = self._vecs(q)
        nq = q.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        _check(self._lib.cphnsw_b200_exact_search_batch(self._h, _p(q), _u64(nq), _u32(k), _p(ids), _p(dist)))
        return ids, dist

    def rerank_batch(self, q, cand, k):
        """The k best of cand[nq][num_cand] by (-<q,x>, id)."""
        q = self._vecs(q)
        cand = np.ascontiguousarray(cand, np.uint32)
        nq = q.shape[0]
        if cand.ndim != 2 or cand.shape[0] != nq:
            raise ValueError("cand must be [nq][num_cand]")
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        _check(self._lib.cphnsw_b200_rerank_batch(self._h, _p(q), _u64(nq), _p(cand), _u32(cand.shape[1]), _u32(k), _p(ids),
                                                  _p(dist)))
        return ids, dist

    def exact_search_dev(self, d_base, n, d_q, nq, k, d_ids, d_dists, stream=0):
        _check(self._lib.cphnsw_b200_exact_search_dev(self._h, C.c_void_p(d_base), _u64(n), C.c_void_p(d_q), _u64(nq), _u32(k),
                                                      C.c_void_p(d_ids), C.c_void_p(d_dists), C.c_void_p(stream)))

    def verify_connectivity(self):
        """Number of nodes reachable from the entry nodes along the directed adjacency."""
        out = C.c_uint64()
        _check(self._lib.cphnsw_b200_verify_connectivity(self._h, C.byref(out)))
        return int(out.value)

    def calibrate(self, num_samples=1000, seed=42):
        """Least-squares fit of the exact distance against the CP score over sampled node pairs:
        (alpha, beta, r_squared)."""
        a, b, r = C.c_double(), C.c_double(), C.c_double()
        _check(self._lib.cphnsw_b200_calibrate(self._h, _u64(num_samples), _u64(seed), C.byref(a), C.byref(b), C.byref(r)))
        return a.value, b.value, r.value

    def get_calibration(self):
        a, b, r, m = C.c_double(), C.c_double(), C.c_double(), C.c_uint64()
        _check(self._lib.cphnsw_b200_get_calibration(self._h, C.byref(a), C.byref(b), C.byref(r), C.byref(m)))
        return a.value, b.value, r.value, int(m.value)

    def search_calibrated_batch(self, q, k, ef, rerank_k=0):
        q = self._vecs(q)
        nq = q.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        _check(self._lib.cphnsw_b200_search_calibrated_batch(self._h, _p(q), _u64(nq), _u32(k), _u32(ef), _u32(rerank_k),
                                                             _p(ids), _p(dist)))
        return ids, dist

    def search_multiprobe_batch(self, q, k, ef, num_probes):
        q = self._vecs(q)
        nq = q.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        _check(self._lib.cphnsw_b200_search_multiprobe_batch(self._h, _p(q), _u64(nq), _u32(k), _u32(ef),
                                                             _u32(num_probes), _p(ids), _p(dist)))
        return ids, dist

    def search_multiprobe(self, q, k, ef, num_probes):
        ids, dist = self.search_multiprobe_batch(q, k, ef, num_probes)
        return self._results(ids[0], dist[0])

    def probe_codes(self, q, num_probes):
        q = self._vecs(q)
        out = np.empty((q.shape[0], num_probes, self.K), self.code_dtype)
        _check(self._lib.cphnsw_b200_probe_codes(self._h, _p(q), _u64(q.shape[0]), _u32(num_probes), _p(out)))
        return out

    @staticmethod
    def _results(ids, dist):
        return [(int(i), float(d)) for i, d in zip(ids, dist) if i != INVALID_NODE]

    def search(self, q, k, ef):
        """One query -> list of (id, distance) ascending (std::vector<SearchResult>)."""
        ids, dist = self.search_batch(q, k, ef)
        return self._results(ids[0], dist[0])

    def search_and_rerank(self, q, k, ef, rerank_k):
        ids, dist = self.search_and_rerank_batch(q, k, ef, rerank_k)
        return self._results(ids[0], dist[0])

    # ---- device-pointer forms (integers are raw device addresses, e.g. torch.Tensor.data_ptr()) ----
    def encode_dev(self, d_x, n, d_codes, d_rotated=0, d_magnitudes=0, stream=0):
        _check(self._lib.cphnsw_b200_encode_dev(self._h, C.c_void_p(d_x), _u64(n), C.c_void_p(d_codes),
                                                C.c_void_p(d_rotated), C.c_void_p(d_magnitudes), C.c_void_p(stream)))

    def code_distance_dev(self, d_a, na, d_b, nb, d_out, stream=0):
        _check(self._lib.cphnsw_b200_code_distance_dev(self._h, C.c_void_p(d_a), _u64(na), C.c_void_p(d_b), _u64(nb),
                                                       C.c_void_p(d_out), C.c_void_p(stream)))

    def knn_graph_dev(self, d_codes, n, k, row_begin, row_end, d_nbrs, d_dist=0, stream=0):
        _check(self._lib.cphnsw_b200_knn_graph_dev(self._h, C.c_void_p(d_codes), _u64(n), _u32(k), _u64(row_begin),
                                                   _u64(row_end), C.c_void_p(d_nbrs), C.c_void_p(d_dist),
                                                   C.c_void_p(stream)))

    def select_neighbors_dev(self, d_codes, n, d_cand, k, row_begin, row_end, M, keep_pruned, d_adj, stream=0):
        _check(self._lib.cphnsw_b200_select_neighbors_dev(self._h, C.c_void_p(d_codes), _u64(n), C.c_void_p(d_cand),
                                                          _u32(k), _u64(row_begin), _u64(row_end), _u32(M),
                                                          C.c_int(int(keep_pruned)), C.c_void_p(d_adj),
                                                          C.c_void_p(stream)))

    def rank_reorder_dev(self, d_cand, n, k, row_begin, row_end, M, alpha, d_kept, stream=0):
        _check(self._lib.cphnsw_b200_rank_reorder_dev(self._h, C.c_void_p(d_cand), _u64(n), _u32(k), _u64(row_begin),
                                                      _u64(row_end), _u32(M), C.c_float(alpha), C.c_void_p(d_kept),
                                                      C.c_void_p(stream)))

    def rank_merge_dev(self, d_kept, n, M, row_begin, row_end, d_adj, stream=0):
        _check(self._lib.cphnsw_b200_rank_merge_dev(self._h, C.c_void_p(d_kept), _u64(n), _u32(M), _u64(row_begin),
                                                    _u64(row_end), C.c_void_p(d_adj), C.c_void_p(stream)))

    def install_dev(self, d_vectors, d_codes, d_adj, n, stream=0):
        _check(self._lib.cphnsw_b200_install_dev(self._h, C.c_void_p(d_vectors), C.c_void_p(d_codes),
                                                 C.c_void_p(d_adj), _u64(n), C.c_void_p(stream)))

    def search_dev(self, d_q, nq, k, ef, rerank_k, d_ids, d_dists, d_stats=0, stream=0):
        _check(self._lib.cphnsw_b200_search_dev(self._h, C.c_void_p(d_q), _u64(nq), _u32(k), _u32(ef), _u32(rerank_k),
                                                C.c_void_p(d_ids), C.c_void_p(d_dists), C.c_void_p(d_stats),
                                                C.c_void_p(stream)))

    KERNELS = {"encode": 0, "code_distance": 1, "knn_graph": 2, "select_neighbors": 3, "search": 4}

    def kernel_time(self, kind):
        """(summed device ms, launches) of a kernel family since the last call; needs set_param("profile", 1)."""
        ms = C.c_double()
        cnt = C.c_uint64()
        _check(self._lib.cphnsw_b200_kernel_time(self._h, C.c_int(self.KERNELS[kind]), C.byref(ms), C.byref(cnt)))
        return ms.value, int(cnt.value)

    def check_device_status(self):
        _check(self._lib.cphnsw_b200_check_device_status(self._h))


class ShardedIndex:
    """One index over several GPUs of one box in one process (``cphnsw_b200_sharded_*``): the bulk build
    sharded by row block with NCCL all-gathers in between, batched searches by query block, one replica
    per device.  ``n_gpus = 0`` takes every usable device."""

    SEARCH, RERANK, MULTIPROBE, BRUTE_FORCE, CALIBRATED = range(5)
    STAGES = ("encode", "allgather_codes", "knn_graph", "prune", "allgather_adjacency_vectors", "install")

    def __init__(self, dim, M=32, ef_construction=200, K=32, component_bytes=1, seed=42, fht_convention=FHT_AVX512,
                 n_gpus=0, devices=None, binary=False):
        self._lib = load_library()
        self._s = C.c_void_p()
        dev = None if devices is None else (C.c_int * len(devices))(*devices)
        _check(self._lib.cphnsw_b200_sharded_create(_u64(dim), _u32(K), _u32(component_bytes), _u32(M), _u32(ef_construction),
                                                    _u64(seed), C.c_int(fht_convention), C.c_int(int(binary)), C.c_int(n_gpus),
                                                    dev, C.byref(self._s)))
        self.dim, self.K, self.M, self.component_bytes = dim, K, M, component_bytes

    def close(self):
        if getattr(self, "_s", None) is not None and self._s.value:
            self._lib.cphnsw_b200_sharded_destroy(self._s)
            self._s = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def gpus(self):
        return int(self._lib.cphnsw_b200_sharded_gpus(self._s))

    def size(self):
        return int(self._lib.cphnsw_b200_sharded_size(self._s))

    def replica(self, g=0):
        """The replica on the g-th device as a (non-owning) CPHNSWIndex."""
        idx = CPHNSWIndex.__new__(CPHNSWIndex)
        idx._lib = self._lib
        idx._h = C.c_void_p(self._lib.cphnsw_b200_sharded_replica(self._s, C.c_int(g)))
        idx._borrowed = True
        idx.dim, idx.K, idx.M, idx.component_bytes = self.dim, self.K, self.M, self.component_bytes
        idx.padded_dim = int(self._lib.cphnsw_b200_padded_dim(idx._h))
        idx.code_dtype = np.uint8 if self.component_bytes == 1 else np.uint16
        return idx

    def set_param(self, name, value):
        _check(self._lib.cphnsw_b200_sharded_set_param(self._s, name.encode(), C.c_double(value)))

    def add_batch_parallel(self, x):
        x = np.ascontiguousarray(x, np.float32)
        _check(self._lib.cphnsw_b200_sharded_add_batch_parallel(self._s, _p(x), _u64(x.shape[0])))

    def add_batch(self, x):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, self.dim)
        _check(self._lib.cphnsw_b200_sharded_add_batch(self._s, _p(x), _u64(x.shape[0])))

    def stage_times(self):
        ms = (C.c_double * len(self.STAGES))()
        _check(self._lib.cphnsw_b200_sharded_stage_times(self._s, ms))
        return dict(zip(self.STAGES, [float(v) for v in ms]))

    def search(self, mode, q, k, ef, arg=0, want_stats=False):
        q = np.ascontiguousarray(q, np.float32).reshape(-1, self.dim)
        nq = q.shape[0]
        ids = np.empty((nq, k), np.uint32)
        dist = np.empty((nq, k), np.float32)
        stats = np.zeros((nq, 2), np.uint32) if want_stats else None
        _check(self._lib.cphnsw_b200_sharded_search(self._s, C.c_int(mode), _p(q), _u64(nq), _u32(k), _u32(ef), _u32(arg),
                                                    _p(ids), _p(dist), _p(stats)))
        return (ids, dist, stats) if want_stats else (ids, dist)

    def search_and_rerank_batch(self, q, k, ef, rerank_k, want_stats=False):
        return self.search(self.RERANK, q, k, ef, rerank_k, want_stats)

    def search_batch(self, q, k, ef, want_stats=False):
        return self.search(self.SEARCH, q, k, ef, 0, want_stats)
