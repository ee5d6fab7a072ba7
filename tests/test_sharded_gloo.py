"""Host-side logic of the multi-GPU path on CPU: world-size-2 ``gloo`` ranks run the same sharded
build orchestration the GPU ranks run (``cphnsw_b200.sharded.build_sharded``), with the stage functions
backed by the CPU oracle, and must reproduce the single-process result exactly."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class OracleStages:
    """Stage functions over CPU torch tensors, computed by the oracle (test double of CudaStages)."""

    def __init__(self, O, signs, K, cb):
        self.O, self.signs, self.K, self.cb = O, signs, K, cb

    def encode(self, x):
        import torch
        codes = self.O.encode(x.numpy(), self.K, self.cb, self.signs)
        # two-byte codes travel as int16 tensors, as in CudaStages
        return torch.from_numpy(codes.view(np.int16) if self.cb == 2 else codes)

    def _codes(self, codes_all):
        a = codes_all.numpy()
        return a.view(np.uint16) if self.cb == 2 else a

    def knn(self, codes_all, k, rb, re):
        import torch
        nb, _ = self.O.knn_graph(self._codes(codes_all), k, rb, re)
        return torch.from_numpy(nb.astype(np.int64))

    def select(self, codes_all, cand, k, rb, re, M, keep_pruned):
        import torch
        adj = self.O.select_neighbors(self._codes(codes_all), cand.numpy().astype(np.uint32), M, keep_pruned, row_begin=rb)
        return torch.from_numpy(adj.astype(np.int64))


def _worker(rank, world, port, n, cb, out_dir):
    for p in (os.path.join(ROOT, "sparse-text-kmeans_b200"), os.path.join(ROOT, "oracle")):
        sys.path.insert(0, p)
    import torch
    import torch.distributed as dist
    import oracle as O
    from cphnsw_b200 import sharded, synthetic
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    try:
        base, _ = synthetic.gaussian_mixture(n, 4, 32, 5, 0.3, 77)
        K, M, knn_k = 16, 8, 16
        signs = O.sign_tables(32, K, 42)
        rb, re = sharded.shard_range(n, rank, world)
        stages = OracleStages(O, signs, K, cb)
        codes_all, adj_all = sharded.build_sharded(stages, torch.from_numpy(base[rb:re]), n, rank, world, dist, knn_k, M)
        np.save(os.path.join(out_dir, "codes_%d.npy" % rank), codes_all.numpy())
        np.save(os.path.join(out_dir, "adj_%d.npy" % rank), adj_all.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,cb", [(401, 1), (512, 1), (401, 2)])  # uneven and even row blocks; one- and two-byte codes
def test_sharded_build_equals_single_process(oracle, tmp_path, n, cb):
    import torch.multiprocessing as mp
    from cphnsw_b200 import sharded, synthetic
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n, cb, str(tmp_path)), nprocs=world, join=True)
    base, _ = synthetic.gaussian_mixture(n, 4, 32, 5, 0.3, 77)
    signs = oracle.sign_tables(32, 16, 42)
    codes = oracle.encode(base, 16, cb, signs)
    cand, _ = oracle.knn_graph(codes, 16)
    adj = oracle.select_neighbors(codes, cand, 8, True)
    for r in range(world):
        got = np.load(tmp_path / ("codes_%d.npy" % r))
        assert np.array_equal(got.view(np.uint16) if cb == 2 else got, codes)
        assert np.array_equal(np.load(tmp_path / ("adj_%d.npy" % r)).astype(np.uint32), adj)


def test_shard_ranges_partition_rows():
    from cphnsw_b200 import sharded
    for n in (0, 1, 7, 8, 1000, 1001):
        for world in (1, 2, 3, 8):
            blocks = [sharded.shard_range(n, r, world) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == n
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in blocks]
            assert max(sizes) - min(sizes) <= 1
