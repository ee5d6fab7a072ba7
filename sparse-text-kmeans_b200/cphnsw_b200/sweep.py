"""Batch-size, ef and multiprobe sweeps of the search calls on a synthetic workload, through the host-pointer
API (the loops the reference's evaluation programs run: evaluation/eval_sift.cpp:377-390 ef sweep, :430,469
multiprobe; batch sizes of the largest configuration).  Prints queries/s and recall@10 against exact_search.

    python sparse-text-kmeans_b200/cphnsw_b200/sweep.py C2 [scale]
"""
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import cphnsw_b200 as cp  # noqa: E402
from cphnsw_b200 import sharded, synthetic  # noqa: E402

name = sys.argv[1]; scale = float(sys.argv[2]) if len(sys.argv) > 2 else 1.0
w = synthetic.workload(name, scale)
base, q = w["base"], w["queries"]
n, nq, dim = base.shape[0], q.shape[0], base.shape[1]
idx = cp.CPHNSWIndex(dim, K=32, M=32)
idx.set_param("entry_scan", w["entry_scan"]); idx.set_param("k_entry", w.get("k_entry", 4))
if n > 2_000_000: idx.set_param("build_seed", 65536)
t0 = time.perf_counter(); idx.add_batch_parallel(base); print(f"{name} n={n} nq={nq}: build {time.perf_counter()-t0:.2f} s", flush=True)
nq_gt = min(nq, 10000)
ids = np.empty((nq_gt, 10), np.uint32)
d_base = torch.from_numpy(base).cuda(); d_q = torch.from_numpy(q[:nq_gt]).cuda()
d_gt = torch.empty((nq_gt, 10), dtype=torch.int32, device="cuda"); d_gd = torch.empty((nq_gt, 10), dtype=torch.float32, device="cuda")
torch.cuda.synchronize(); t0 = time.perf_counter()
idx.exact_search_dev(d_base.data_ptr(), n, d_q.data_ptr(), nq_gt, 10, d_gt.data_ptr(), d_gd.data_ptr()); torch.cuda.synchronize()
print(f"ground truth {nq_gt} x {n}: {(time.perf_counter()-t0)*1e3:.0f} ms", flush=True)
gt = d_gt.cpu().numpy().view(np.uint32).astype(np.int64); del d_base
def run(fn, batch, limit):
    """queries/s through the host API (host buffers in and out) and the ids of the first nq_gt queries"""
    m = min(nq, limit); out = []
    fn(q[:min(batch, m)])  # warm
    t0 = time.perf_counter()
    for s in range(0, m, batch): out.append(fn(q[s:min(m, s + batch)])[0])
    dt = time.perf_counter() - t0
    return m / dt, np.concatenate(out)
print("batch sweep (search_and_rerank k=10 ef=100 rerank_k=500, host buffers):")
for batch, limit in ((1, 300), (64, 6400), (1024, 20480), (10000, nq), (nq, nq)):
    qps, got = run(lambda x: idx.search_and_rerank_batch(x, 10, 100, 500), batch, limit)
    m = min(len(got), nq_gt)
    print(f"  batch {batch:6d}: {qps:10.0f} queries/s ({1e3*batch/qps:8.3f} ms per call) recall@10 {sharded.recall_at_k(got[:m], gt[:m], 10):.4f}", flush=True)
print("ef sweep, search_and_rerank rerank_k=500, batch 10000 (beam = max(ef, rerank_k)):")
for ef in (50, 100, 200, 400):
    qps, got = run(lambda x: idx.search_and_rerank_batch(x, 10, ef, 500), 10000, nq_gt)
    print(f"  ef {ef:4d}: {qps:10.0f} queries/s recall@10 {sharded.recall_at_k(got, gt, 10):.4f}", flush=True)
print("ef sweep, rerank_k = ef:")
for ef in (50, 100, 200, 400):
    qps, got = run(lambda x: idx.search_and_rerank_batch(x, 10, ef, ef), 10000, nq_gt)
    print(f"  ef {ef:4d}: {qps:10.0f} queries/s recall@10 {sharded.recall_at_k(got, gt, 10):.4f}", flush=True)
print("ef sweep, search without rerank:")
for ef in (50, 100, 200, 400):
    qps, got = run(lambda x: idx.search_batch(x, 10, ef), 10000, nq_gt)
    print(f"  ef {ef:4d}: {qps:10.0f} queries/s recall@10 {sharded.recall_at_k(got, gt, 10):.4f}", flush=True)
print("search_multiprobe, ef=100, batch 10000:")
for T in (1, 4, 16):
    qps, got = run(lambda x: idx.search_multiprobe_batch(x, 10, 100, T), 10000, nq_gt)
    print(f"  probes {T:3d}: {qps:10.0f} queries/s recall@10 {sharded.recall_at_k(got, gt, 10):.4f}", flush=True)
