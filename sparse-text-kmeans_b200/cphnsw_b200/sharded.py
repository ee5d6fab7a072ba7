"""Row-block sharding of the index build and query-block sharding of the search across the GPUs of
one box, one process per GPU.

The build shards by contiguous row blocks: every rank encodes its own rows, the codes are
all-gathered (32 B per vector at K=32 - the only data the distance stage needs from other ranks),
every rank computes the kNN rows and the pruned adjacency rows of its block against the replicated
codes, and the adjacency rows are all-gathered so that every rank can install the whole index.
Searching needs no communication: queries are split across ranks, the index is replicated.

The collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo on CPU).  The stage
functions are injected, so the same orchestration runs on device tensors with the CUDA library and
on CPU tensors in the host-side tests.
"""
import numpy as np


def shard_range(n, rank, world):
    """Contiguous block [begin, end) of ``n`` rows owned by ``rank``; blocks differ by at most one row."""
    base, rem = divmod(n, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def all_gather_rows(local, n, rank, world, dist=None):
    """All-gathers row blocks laid out by ``shard_range`` into one [n, ...] tensor on every rank."""
    import torch
    if world == 1:
        return local
    if local.dtype == torch.int16:
        # NCCL's torch binding moves no 16-bit integers (two-byte codes): the rows travel as bytes
        as_bytes = local.contiguous().view(torch.uint8)
        return all_gather_rows(as_bytes, n, rank, world, dist).view(torch.int16)
    counts = [shard_range(n, r, world)[1] - shard_range(n, r, world)[0] for r in range(world)]
    width = max(counts)
    out = torch.empty((world * width,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    if all(c == width for c in counts):  # equal blocks travel as they are
        dist.all_gather_into_tensor(out, local.contiguous())
        return out
    pad = torch.zeros((width,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    dist.all_gather_into_tensor(out, pad)
    return torch.cat([out[r * width: r * width + counts[r]] for r in range(world)], dim=0)


def build_sharded(stages, vectors_local, n, rank, world, dist, knn_k, M, keep_pruned=True, timers=None):
    """Runs encode -> all-gather(codes) -> kNN rows -> select rows -> all-gather(adjacency).

    ``stages`` provides ``encode(x_local) -> codes_local``, ``knn(codes_all, k, rb, re) -> cand`` and
    ``select(codes_all, cand, k, rb, re, M, keep_pruned) -> adj_local`` on tensors.
    ``timers(name)`` (optional) returns a context manager used to time each stage.
    Returns (codes_all, adj_all).
    """
    import contextlib
    tm = timers or (lambda name: contextlib.nullcontext())
    rb, re = shard_range(n, rank, world)
    assert vectors_local.shape[0] == re - rb
    if hasattr(stages, "reserve"):  # output buffers exist before any stage is timed
        stages.reserve(re - rb, knn_k, M, vectors_local.device)
    with tm("encode"):
        codes_local = stages.encode(vectors_local)
    with tm("allgather_codes"):
        codes_all = all_gather_rows(codes_local, n, rank, world, dist)
    with tm("knn_graph"):
        cand = stages.knn(codes_all, knn_k, rb, re)
    with tm("select_neighbors"):
        adj_local = stages.select(codes_all, cand, knn_k, rb, re, M, keep_pruned)
    with tm("allgather_adjacency"):
        adj_all = all_gather_rows(adj_local, n, rank, world, dist)
    return codes_all, adj_all


class CudaStages:
    """Stage functions over torch CUDA tensors, backed by the ``_dev`` entry points of the C ABI."""

    def __init__(self, index):
        self.index = index
        self._buf = {}

    def reserve(self, rows, k, M, device):
        """Allocates the stage outputs for `rows` local rows, so that a timed stage does not pay for the allocation."""
        import torch
        ct = torch.uint8 if self.index.component_bytes == 1 else torch.int16
        self._buf = {"codes": torch.empty((rows, self.index.K), dtype=ct, device=device),
                     "cand": torch.empty((rows, k), dtype=torch.int32, device=device),
                     "adj": torch.empty((rows, M), dtype=torch.int32, device=device)}
        torch.cuda.synchronize(device)

    def _out(self, name, shape, dtype, device):
        import torch
        b = self._buf.pop(name, None)
        if b is not None and tuple(b.shape) == tuple(shape) and b.dtype == dtype and b.device == device:
            return b
        return torch.empty(shape, dtype=dtype, device=device)

    def encode(self, x):
        import torch
        ct = torch.uint8 if self.index.component_bytes == 1 else torch.int16
        codes = self._out("codes", (x.shape[0], self.index.K), ct, x.device)
        self.index.encode_dev(x.data_ptr(), x.shape[0], codes.data_ptr())
        return codes

    def knn(self, codes_all, k, rb, re):
        import torch
        cand = self._out("cand", (re - rb, k), torch.int32, codes_all.device)
        self.index.knn_graph_dev(codes_all.data_ptr(), codes_all.shape[0], k, rb, re, cand.data_ptr())
        return cand

    def select(self, codes_all, cand, k, rb, re, M, keep_pruned):
        import torch
        adj = self._out("adj", (re - rb, M), torch.int32, codes_all.device)
        self.index.select_neighbors_dev(codes_all.data_ptr(), codes_all.shape[0], cand.data_ptr(), k, rb, re, M,
                                        keep_pruned, adj.data_ptr())
        return adj


def split_queries(nq, rank, world):
    return shard_range(nq, rank, world)


def recall_at_k(found, truth, k):
    """|retrieved ∩ truth| / k averaged over queries (evaluation/metrics/recall.hpp:22-39)."""
    found = np.asarray(found)[:, :k]
    truth = np.asarray(truth)[:, :k]
    hits = 0
    for f, t in zip(found, truth):
        hits += len(set(f.tolist()) & set(t.tolist()))
    return hits / float(truth.shape[0] * k)
