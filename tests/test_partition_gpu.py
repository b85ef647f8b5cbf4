"""GPU parity of the stable partition-by-owner kernels (first step of every DISTRIBUTED op)
against the CPU oracle's bucket rule, through the C ABI."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_partition(wgb, torch, idx_t, first_row, entry="wholegraph_b200_partition_by_owner"):
    lib = wgb.lib()
    world = len(first_row) - 1
    n = idx_t.numel()
    ws_bytes = lib.wholegraph_b200_partition_workspace_bytes(n, world)
    ws = torch.empty(max(ws_bytes, 8), dtype=torch.uint8, device="cuda")
    sorted_ids = torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda")
    positions = torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda")
    counts = torch.full((world,), -7, dtype=torch.int64, device="cuda")
    starts = torch.full((world,), -7, dtype=torch.int64, device="cuda")
    fr = (C.c_int64 * (world + 1))(*[int(x) for x in first_row])
    rc = getattr(lib, entry)(C.c_void_p(idx_t.data_ptr()), 1 if idx_t.dtype == torch.int64 else 0, n, fr, world,
                             C.c_void_p(ws.data_ptr()), ws_bytes, C.c_void_p(sorted_ids.data_ptr()),
                             C.c_void_p(positions.data_ptr()), C.c_void_p(counts.data_ptr()),
                             C.c_void_p(starts.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    wgb.check(rc, entry)
    torch.cuda.synchronize()
    return sorted_ids.cpu().numpy(), positions.cpu().numpy(), counts.cpu().numpy(), starts.cpu().numpy()


def check_against_oracle(orc, idx, first_row, sorted_ids, positions, counts, starts):
    world = len(first_row) - 1
    rows = first_row[-1]
    want_counts, _, _ = orc.bucket_sort_ids(np.where(idx >= rows, -1, idx), np.asarray(first_row, dtype=np.int64))
    assert np.array_equal(counts, want_counts)
    assert np.array_equal(starts, np.concatenate([[0], np.cumsum(want_counts)[:-1]]))
    idx64 = idx.astype(np.int64)
    for r in range(world):
        seg = slice(int(starts[r]), int(starts[r] + counts[r]))
        pos = positions[seg]
        # stable: list order kept inside the group, and exactly the ids this rank owns
        assert np.all(np.diff(pos) > 0)
        owned = np.nonzero((idx64 >= first_row[r]) & (idx64 < first_row[r + 1]))[0]
        assert np.array_equal(pos, owned)
        assert np.array_equal(sorted_ids[seg], idx64[pos])


@pytest.mark.parametrize("world", [1, 2, 3, 8, 64])
@pytest.mark.parametrize("n", [0, 1, 255, 2048, 2049, 100_003])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_partition_equal_split(gpu, wgb, orc, world, n, idx_dtype):
    import torch
    rng = np.random.default_rng(world * 1000 + n)
    rows = 1_000_003
    first_row = [int(x) for x in orc.equal_partition_offsets(rows, world)]
    idx = rng.integers(0, rows, size=n).astype(idx_dtype)
    if n > 8:
        idx[rng.integers(0, n, size=n // 10)] = -1          # skipped by every op
        idx[rng.integers(0, n, size=3)] = rows + 5          # past the end: dropped as well
    out = run_partition(wgb, torch, torch.from_numpy(idx).cuda(), first_row)
    check_against_oracle(orc, idx, first_row, *out)


def test_partition_custom_split_and_skew(gpu, wgb, orc):
    import torch
    rng = np.random.default_rng(3)
    first_row = [0, 10, 11, 5000, 5000 + 1, 900_000]  # very uneven shards
    idx = np.concatenate([rng.integers(0, 900_000, size=50_000), np.full(30_000, 10), rng.integers(0, 11, size=5_000)])
    rng.shuffle(idx)
    idx = idx.astype(np.int64)
    out = run_partition(wgb, torch, torch.from_numpy(idx).cuda(), first_row)
    check_against_oracle(orc, idx, first_row, *out)
