"""The multi-GPU index behind the C ABI (cphnsw_b200_sharded_*): one process, one replica per device, NCCL
all-gathers between the build stages.  With one device it must be the plain index; with two or more the
adjacency must be the single-device adjacency bit for bit and searches must return the same arrays.  The
multi-device cases run where the box has the devices (they are skipped on a one-GPU box)."""
import numpy as np
import pytest

from cphnsw_b200 import synthetic

pytestmark = pytest.mark.gpu


def single(cp, base, **params):
    idx = cp.CPHNSWIndex(base.shape[1], M=32, ef_construction=200, K=32, component_bytes=1)
    for name, v in params.items():
        idx.set_param(name, v)
    idx.add_batch_parallel(base)
    return idx


@pytest.mark.parametrize("gpus", [1, 2, 4])
@pytest.mark.parametrize("n", [6000, 6001])  # equal blocks (one all-gather) and unequal ones (grouped broadcasts)
def test_sharded_build_and_search_equal_single_device(cp, gpus, n):
    if cp.device_count() < gpus:
        pytest.skip("needs %d GPUs" % gpus)
    base, q = synthetic.gaussian_mixture(n, 300, 128, 12, 0.3, 31)
    ref = single(cp, base, entry_scan=256, k_entry=8)
    sh = cp.ShardedIndex(128, n_gpus=gpus)
    sh.set_param("entry_scan", 256)
    sh.set_param("k_entry", 8)
    sh.add_batch_parallel(base)
    assert sh.gpus() == gpus and sh.size() == n
    for g in range(gpus):
        rep = sh.replica(g)
        assert np.array_equal(rep.codes(), ref.codes())
        assert np.array_equal(rep.adjacency(), ref.adjacency())
    want = ref.search_and_rerank_batch(q, 10, 100, 200, want_stats=True)
    got = sh.search_and_rerank_batch(q, 10, 100, 200, want_stats=True)  # 300 queries: split across the replicas
    assert all(np.array_equal(a, b) for a, b in zip(got, want))
    got1 = sh.search_and_rerank_batch(q[:5], 10, 100, 200)            # a small batch goes to one replica
    assert np.array_equal(got1[0], want[0][:5]) and np.array_equal(got1[1], want[1][:5])
    ws = ref.search_batch(q, 10, 64)
    gs = sh.search_batch(q, 10, 64)
    assert np.array_equal(gs[0], ws[0]) and np.array_equal(gs[1], ws[1])
    wm = ref.search_multiprobe_batch(q[:100], 10, 50, 4)
    gm = sh.search(sh.MULTIPROBE, q[:100], 10, 50, 4)
    assert np.array_equal(gm[0], wm[0]) and np.array_equal(gm[1], wm[1])
    t = sh.stage_times()
    assert (t["knn_graph"] > 0) == (gpus > 1)  # one device: the replica's own add_batch_parallel does the work
    # incremental insertion keeps the replicas identical
    more, _ = synthetic.gaussian_mixture(500, 1, 128, 12, 0.3, 32)
    sh.add_batch(more)
    ref.add_batch(more)
    for g in range(gpus):
        assert np.array_equal(sh.replica(g).adjacency(), ref.adjacency())


@pytest.mark.parametrize("gpus", [1, 2])
def test_sharded_rank_prune_and_unpruned_builds(cp, gpus):
    if cp.device_count() < gpus:
        pytest.skip("needs %d GPUs" % gpus)
    base, _ = synthetic.gaussian_mixture(5000, 1, 128, 10, 0.3, 33)
    for params in ({"rank_prune": 1, "rank_pruning_alpha": 1.1}, {"prune": 0}, {"knn_k": 40}):
        ref = single(cp, base, **params)
        sh = cp.ShardedIndex(128, n_gpus=gpus)
        for name, v in params.items():
            sh.set_param(name, v)
        sh.add_batch_parallel(base)
        for g in range(gpus):
            assert np.array_equal(sh.replica(g).adjacency(), ref.adjacency()), params


def test_sharded_bad_arguments(cp):
    with pytest.raises((ValueError, cp.CPHNSWError)):
        cp.ShardedIndex(128, n_gpus=cp.device_count() + 1)
    with pytest.raises(ValueError):
        cp.ShardedIndex(128, n_gpus=1, devices=[cp.device_count() + 3])
    sh = cp.ShardedIndex(128, n_gpus=1)
    with pytest.raises(cp.CPHNSWError):
        sh.search_batch(np.zeros((1, 128), np.float32), 10, 10)  # empty index
    with pytest.raises(ValueError):
        sh.search(9, np.zeros((1, 128), np.float32), 10, 10)
