"""Seeded synthetic stand-ins for the datasets the reference measures on (SIFT-1M: 1M x 128 with
10k queries; GIST-1M: 1M x 960 non-negative).  Shapes and value ranges follow those datasets;
no item of them is reproduced.  All vectors are float32 and L2-normalised with the
``norm > 1e-10`` guard of evaluation/datasets/dataset_loader.hpp:225-240.
"""
import os

import numpy as np


def normalize(x):
    x = np.ascontiguousarray(x, np.float32)
    norm = np.sqrt((x.astype(np.float32) ** 2).sum(axis=1, dtype=np.float32))
    scale = np.where(norm > 1e-10, 1.0 / np.maximum(norm, 1e-30), 1.0).astype(np.float32)
    return (x * scale[:, None]).astype(np.float32)


def gaussian_sphere(n, nq, dim, seed, query_stream=0):
    """i.i.d. N(0,1) per coordinate, then normalised (the random-sphere generator of
    dataset_loader.hpp:145-185 with numpy streams).  ``query_stream`` selects an independent query set."""
    base = normalize(np.random.default_rng([seed, 1]).standard_normal((n, dim), dtype=np.float32))
    queries = normalize(np.random.default_rng([seed, 2, query_stream]).standard_normal((nq, dim), dtype=np.float32))
    return base, queries


def gaussian_mixture(n, nq, dim, n_clusters, sigma, seed, query_stream=0, chunk=1 << 18):
    """Uniform-weight mixture: centres ~ N(0,1) per coordinate, points = centre + sigma*N(0,1),
    normalised; queries from the same mixture with an independent stream."""
    rng = np.random.default_rng(seed)
    centres = rng.standard_normal((n_clusters, dim), dtype=np.float32)

    def draw(m, stream):
        out = np.empty((m, dim), np.float32)
        for i0 in range(0, m, chunk):
            i1 = min(m, i0 + chunk)
            a = stream.integers(0, n_clusters, i1 - i0)
            out[i0:i1] = normalize(centres[a] + np.float32(sigma) * stream.standard_normal((i1 - i0, dim), dtype=np.float32))
        return out

    base = draw(n, np.random.default_rng([seed, 1]))
    queries = draw(nq, np.random.default_rng([seed, 2, query_stream]))
    return base, queries


def abs_gaussian(n, nq, dim, seed, query_stream=0, chunk=1 << 16):
    """Non-negative |N(0,1)| coordinates, normalised (GIST-like value range)."""
    def draw(m, stream):
        out = np.empty((m, dim), np.float32)
        for i0 in range(0, m, chunk):
            i1 = min(m, i0 + chunk)
            out[i0:i1] = normalize(np.abs(stream.standard_normal((i1 - i0, dim), dtype=np.float32)))
        return out

    return draw(n, np.random.default_rng([seed, 1])), draw(nq, np.random.default_rng([seed, 2, query_stream]))


def abs_mixture(n, nq, dim, n_clusters, sigma, seed, query_stream=0, chunk=1 << 16):
    """Non-negative clustered vectors (GIST-like: every coordinate >= 0, so all vectors share one orthant and a
    large common component, with neighbourhood structure on top): centres |N(0,1)| per coordinate, points =
    |centre + sigma*N(0,1)|, normalised; queries from the same mixture with an independent stream."""
    rng = np.random.default_rng(seed)
    centres = np.abs(rng.standard_normal((n_clusters, dim), dtype=np.float32))

    def draw(m, stream):
        out = np.empty((m, dim), np.float32)
        for i0 in range(0, m, chunk):
            i1 = min(m, i0 + chunk)
            a = stream.integers(0, n_clusters, i1 - i0)
            out[i0:i1] = normalize(np.abs(centres[a] + np.float32(sigma) * stream.standard_normal((i1 - i0, dim), dtype=np.float32)))
        return out

    return draw(n, np.random.default_rng([seed, 1])), draw(nq, np.random.default_rng([seed, 2, query_stream]))


# The five benchmark workloads (full sizes) and a clustered variant of the third; ``scale`` shrinks base, queries and clusters together
# so that cluster populations stay the same.
def workload(name, scale=1.0, query_stream=0):
    """``query_stream`` picks an independent query set from the same distribution (one per rank)."""
    s = float(scale)
    qs = query_stream

    def sz(v, lo=1):
        return max(lo, int(round(v * s)))

    if name == "C1":
        base, q = gaussian_sphere(sz(100_000), sz(1_000, 10), 128, 0, qs)
        return dict(name="C1", base=base, queries=q, K=32, component_bytes=1, M=32, ef_construction=200,
                    k=10, ef=100, rerank_k=500, entry_scan=4)
    if name == "C2":
        base, q = gaussian_mixture(sz(1_000_000), sz(10_000, 10), 128, sz(1_000), 0.3, 1, qs)
        return dict(name="C2", base=base, queries=q, K=32, component_bytes=1, M=32, ef_construction=200,
                    k=10, ef=100, rerank_k=500, entry_scan=sz(8_192, 4), k_entry=32)
    if name == "C3":
        base, q = abs_gaussian(sz(1_000_000), sz(10_000, 10), 960, 2, qs)
        return dict(name="C3", base=base, queries=q, K=32, component_bytes=2, M=32, ef_construction=200,
                    k=10, ef=200, rerank_k=1000, entry_scan=4)
    if name == "C3c":
        # the shape and parameters of C3 on vectors that have neighbourhoods (independent coordinates have none: every
        # pair sits at cosine ~0.64 and no index can rank them): 1,000 clusters and, as for C2, an entry scan
        base, q = abs_mixture(sz(1_000_000), sz(10_000, 10), 960, sz(1_000), 0.3, 2, qs)
        return dict(name="C3c", base=base, queries=q, K=32, component_bytes=2, M=32, ef_construction=200,
                    k=10, ef=200, rerank_k=1000, entry_scan=sz(8_192, 4), k_entry=32)
    if name == "C4":
        base, q = gaussian_mixture(sz(10_000_000), sz(1_000, 10), 96, sz(10_000), 0.25, 3, qs)
        return dict(name="C4", base=base, queries=q, K=32, component_bytes=1, M=32, ef_construction=200,
                    k=10, ef=100, rerank_k=500, knn_k=32, entry_scan=sz(65_536, 4), k_entry=32)
    if name == "C5":
        base, q = gaussian_mixture(sz(10_000_000), sz(100_000, 10), 128, sz(1_000), 0.3, 4, qs)
        return dict(name="C5", base=base, queries=q, K=32, component_bytes=1, M=32, ef_construction=200,
                    k=10, ef=100, rerank_k=500, entry_scan=sz(8_192, 4), k_entry=32)
    raise ValueError("unknown workload %r" % name)


def workload_from_files(base_path, query_path, max_base=0, max_queries=0, rank=0, world=1):
    """A workload from fvecs files (e.g. sift_base.fvecs / sift_query.fvecs when they are available):
    rows normalised to unit length like the reference's load_*_normalized loaders do
    (evaluation/datasets/dataset_loader.hpp:225-240), parameters of the C2 configuration (uint16
    components when the padded dimension exceeds 128).  Queries are split across ranks."""
    from . import vecs_io
    base = vecs_io.normalize_rows(vecs_io.read_fvecs(base_path, max_base))
    q = vecs_io.normalize_rows(vecs_io.read_fvecs(query_path, max_queries))
    if q.shape[1] != base.shape[1]:
        raise ValueError("Query dimension mismatch")  # dataset_loader.hpp:130-132
    q = np.ascontiguousarray(q[rank::world])
    wide = base.shape[1] > 128
    return dict(name="files:" + os.path.basename(base_path), base=base, queries=q, K=32, component_bytes=2 if wide else 1,
                M=32, ef_construction=200, k=10, ef=200 if wide else 100, rerank_k=1000 if wide else 500,
                entry_scan=8192, k_entry=32)

