"""The allocation-free code-distance entry point (``cphnsw_b200_code_distance_noalloc``).

It exists for hosts that must not allocate device memory while running (fixed memory plans,
plugins living inside another allocator, latency paths that cannot afford cudaMalloc's implicit
synchronisation): its scratch is an array built into the library instead of a buffer grown on
demand.  The test feeds it device buffers owned by the test itself and checks, on two calls in a
row that share that built-in scratch, that it returns exactly what the ordinary device entry point
returns (integer distances: bit-exact).  The second call is smaller and has a different code shape
than the first, so anything it wrongly kept from the first call would show.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _device_arrays(torch, a, b):
    dev = torch.device("cuda", 0)
    ta = torch.from_numpy(a.view(np.uint8).reshape(a.shape[0], -1)).to(dev)
    tb = torch.from_numpy(b.view(np.uint8).reshape(b.shape[0], -1)).to(dev)
    out = torch.full((a.shape[0], b.shape[0]), -1, dtype=torch.int16, device=dev)
    return ta, tb, out


def _both_ways(cp, torch, K, cb, na, nb, seed, check_memory=False):
    rng = np.random.default_rng(seed)
    dt = np.uint8 if cb == 1 else np.uint16
    hi = 256 if cb == 1 else 2048
    a = rng.integers(0, hi, (na, K)).astype(dt)
    b = rng.integers(0, hi, (nb, K)).astype(dt)
    m = min(na, nb)
    b[:m] = np.where(rng.random((m, K)) < 0.5, a[:m], b[:m])  # plenty of equal components
    ta, tb, out_new = _device_arrays(torch, a, b)
    _, _, out_ref = _device_arrays(torch, a, b)
    idx = cp.CPHNSWIndex(128 if cb == 1 else 1024, K=K, component_bytes=cb)
    idx.code_distance_dev(ta.data_ptr(), na, tb.data_ptr(), nb, out_ref.data_ptr())
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(0)[0] if check_memory else None
    cp.code_distance_noalloc(ta.data_ptr(), na, tb.data_ptr(), nb, K, cb, out_new.data_ptr())
    torch.cuda.synchronize()
    if check_memory:
        # the device's free memory is what it was: the call allocated nothing (the first call on a device may
        # make the driver load the kernels it uses, so the claim is checked from the second call on)
        assert torch.cuda.mem_get_info(0)[0] == free_before
    want = (a[:, None, :] != b[None, :, :]).sum(-1).astype(np.int16)
    return out_new.cpu().numpy(), out_ref.cpu().numpy(), want


def test_noalloc_matches_existing_entry_point_twice_in_a_row(cp):
    import torch
    torch.cuda.set_device(0)
    # first call: odd row width (padding path), fills a good part of the built-in scratch
    new1, ref1, want1 = _both_ways(cp, torch, K=13, cb=2, na=3000, nb=5000, seed=1)
    assert np.array_equal(new1, ref1)
    assert np.array_equal(new1, want1)
    # second call straight after: smaller, other component type and width
    new2, ref2, want2 = _both_ways(cp, torch, K=32, cb=1, na=257, nb=1000, seed=2, check_memory=True)
    assert np.array_equal(new2, ref2)
    assert np.array_equal(new2, want2)


def test_noalloc_rejects_oversized_and_bad_arguments(cp):
    import torch
    torch.cuda.set_device(0)
    buf = torch.zeros(64, dtype=torch.uint8, device="cuda:0")
    # 1 MiB of scratch holds 32,768 rows of 32 bytes: one more row must be refused, before any launch
    with pytest.raises(ValueError) as e:
        cp.code_distance_noalloc(buf.data_ptr(), 32768, buf.data_ptr(), 1, 32, 1, buf.data_ptr())
    assert "scratch" in str(e.value)
    with pytest.raises(ValueError):
        cp.code_distance_noalloc(buf.data_ptr(), 1, buf.data_ptr(), 1, 0, 1, buf.data_ptr())
    with pytest.raises(ValueError):
        cp.code_distance_noalloc(buf.data_ptr(), 1, buf.data_ptr(), 1, 32, 3, buf.data_ptr())
    with pytest.raises(ValueError):
        cp.code_distance_noalloc(0, 1, buf.data_ptr(), 1, 32, 1, buf.data_ptr())
    # empty inputs are a no-op
    cp.code_distance_noalloc(buf.data_ptr(), 0, buf.data_ptr(), 5, 32, 1, buf.data_ptr())
