"""The allocation-free partition entry point against the regular one.

wholegraph_b200_partition_by_owner_no_alloc serves callers that may not touch the CUDA
allocator while they run (all device memory already given to their own pool, or no room for the
device-wide stall of a cudaMalloc) and so cannot provide a workspace: its scratch is a fixed
array inside the library.  Here it is called twice in a row through the C ABI, on different
request lists, and every output must equal the regular entry point's bit for bit; the second
call also shows that what the first one left in the shared array does no harm.  Requests
beyond the array's size must be refused.  The file name sorts last so that a run stopping at
the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _outputs(torch, n, world):
    return (torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda"),
            torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda"),
            torch.full((world,), -7, dtype=torch.int64, device="cuda"),
            torch.full((world,), -7, dtype=torch.int64, device="cuda"))


def _regular(wgb, torch, idx_t, first_row):
    lib = wgb.lib()
    world, n = len(first_row) - 1, idx_t.numel()
    ws_bytes = lib.wholegraph_b200_partition_workspace_bytes(n, world)
    ws = torch.empty(max(ws_bytes, 8), dtype=torch.uint8, device="cuda")
    outs = _outputs(torch, n, world)
    fr = (C.c_int64 * (world + 1))(*first_row)
    wgb.check(lib.wholegraph_b200_partition_by_owner(
        C.c_void_p(idx_t.data_ptr()), 1 if idx_t.dtype == torch.int64 else 0, n, fr, world,
        C.c_void_p(ws.data_ptr()), ws_bytes, *[C.c_void_p(o.data_ptr()) for o in outs],
        C.c_void_p(torch.cuda.current_stream().cuda_stream)), "partition_by_owner")
    torch.cuda.synchronize()
    return [o.cpu().numpy() for o in outs]


def _no_alloc(wgb, torch, idx_t, first_row):
    lib = wgb.lib()
    world, n = len(first_row) - 1, idx_t.numel()
    outs = _outputs(torch, n, world)
    fr = (C.c_int64 * (world + 1))(*first_row)
    rc = lib.wholegraph_b200_partition_by_owner_no_alloc(
        C.c_void_p(idx_t.data_ptr()), 1 if idx_t.dtype == torch.int64 else 0, n, fr, world,
        *[C.c_void_p(o.data_ptr()) for o in outs], C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, [o.cpu().numpy() for o in outs]


def test_no_alloc_partition_matches_regular_entry_twice(gpu, wgb, orc):
    import torch
    rows = 5_000_011
    cases = [(8, 1_000_003, np.int64, 11), (3, 70_001, np.int32, 12)]  # two calls in a row
    for world, n, dt, seed in cases:
        rng = np.random.default_rng(seed)
        first_row = [int(x) for x in orc.equal_partition_offsets(rows, world)]
        idx = rng.integers(0, rows, size=n).astype(dt)
        idx[rng.integers(0, n, size=n // 20)] = -1
        idx_t = torch.from_numpy(idx).cuda()
        want = _regular(wgb, torch, idx_t, first_row)
        rc, got = _no_alloc(wgb, torch, idx_t, first_row)
        assert rc == 0
        used = int(want[2].sum())
        assert np.array_equal(got[2], want[2]) and np.array_equal(got[3], want[3])   # counts, starts
        assert np.array_equal(got[0][:used], want[0][:used])                         # sorted ids
        assert np.array_equal(got[1][:used], want[1][:used])                         # positions


def test_no_alloc_partition_rejects_oversized_requests(gpu, wgb, orc):
    import torch
    world = 64
    n = 2048 * 300  # 300 tiles x 64 ranks = 19,200 histogram words > the built-in 16,508
    first_row = [int(x) for x in orc.equal_partition_offsets(10_000_000, world)]
    idx_t = torch.zeros(n, dtype=torch.int64, device="cuda")
    rc, outs = _no_alloc(wgb, torch, idx_t, first_row)
    assert rc == int(wgb.ErrorCode.INVALID_VALUE)
    assert np.all(outs[2] == -7)  # nothing was launched
