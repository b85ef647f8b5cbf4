"""GPU parity of the request de-duplication (first step of a DISTRIBUTED gather) on one GPU,
through the C ABI: distinct valid ids ascending (hence grouped by owner), the slot of every list
position, and the per-owner group sizes, against the CPU oracle's bucket-and-sort and numpy.
Role of the reference's bucket_and_exchange_ids_func up to the exchange
(cpp/src/wholegraph_tensor_ops/functions/exchange_ids_nccl_func.cu:32-104, :146-215)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_unique(wgb, torch, idx_t, first_row, entry="wholegraph_b200_unique_by_owner"):
    lib = wgb.lib()
    world, n = len(first_row) - 1, idx_t.numel()
    ws_bytes = lib.wholegraph_b200_unique_workspace_bytes(n, first_row[-1])
    ws = torch.empty(max(ws_bytes, 8), dtype=torch.uint8, device="cuda")
    unique_ids = torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda")
    inverse = torch.full((max(n, 1),), -7, dtype=torch.int64, device="cuda")
    counts = torch.full((world,), -7, dtype=torch.int64, device="cuda")
    starts = torch.full((world,), -7, dtype=torch.int64, device="cuda")
    fr = (C.c_int64 * (world + 1))(*[int(x) for x in first_row])
    rc = getattr(lib, entry)(
        C.c_void_p(idx_t.data_ptr()), 1 if idx_t.dtype == torch.int64 else 0, n, fr, world, C.c_void_p(ws.data_ptr()),
        ws_bytes, C.c_void_p(unique_ids.data_ptr()), C.c_void_p(inverse.data_ptr()), C.c_void_p(counts.data_ptr()),
        C.c_void_p(starts.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    wgb.check(rc, entry)
    torch.cuda.synchronize()
    return unique_ids.cpu().numpy(), inverse.cpu().numpy(), counts.cpu().numpy(), starts.cpu().numpy()


def check(orc, idx, first_row, unique_ids, inverse, counts, starts):
    rows, n = first_row[-1], idx.shape[0]
    idx64 = idx.astype(np.int64)
    valid = (idx64 >= 0) & (idx64 < rows)
    want = np.unique(idx64[valid])
    total = int(counts.sum())
    assert total == want.shape[0]
    assert np.array_equal(unique_ids[:total], want)
    # per-owner groups: the oracle's bucket counts of the DISTINCT ids (one request per id)
    want_counts, want_sorted, _ = orc.bucket_sort_ids(want, np.asarray(first_row, dtype=np.int64))
    assert np.array_equal(counts, want_counts)
    assert np.array_equal(starts, np.concatenate([[0], np.cumsum(want_counts)[:-1]]))
    assert np.array_equal(unique_ids[:total], want_sorted[:total])      # ascending ids are already owner-grouped
    if n:
        inv = inverse[:n]
        assert np.all(inv[~valid] == -1)
        assert np.array_equal(unique_ids[inv[valid]], idx64[valid])      # every position finds its own id


@pytest.mark.parametrize("world", [1, 2, 8, 64])
@pytest.mark.parametrize("n", [0, 1, 257, 4096, 100_003])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_unique_by_owner_equal_split(gpu, wgb, orc, world, n, idx_dtype):
    import torch
    rng = np.random.default_rng(world * 977 + n)
    rows = 1_000_003
    first_row = [int(x) for x in orc.equal_partition_offsets(rows, world)]
    idx = rng.integers(0, rows, size=n).astype(idx_dtype)
    if n > 8:
        idx[: n // 3] = idx[n // 3: 2 * (n // 3)]                    # a third of the list repeats another third
        idx[rng.integers(0, n, size=n // 10)] = -1                    # skipped by every op
        idx[rng.integers(0, n, size=3)] = rows + 5                    # past the end: dropped as well
    out = run_unique(wgb, torch, torch.from_numpy(idx).cuda(), first_row)
    check(orc, idx, first_row, *out)


def test_unique_by_owner_skewed_list_and_uneven_shards(gpu, wgb, orc):
    import torch
    rng = np.random.default_rng(5)
    first_row = [0, 10, 11, 5000, 5001, 900_000]
    idx = np.concatenate([rng.integers(0, 900_000, size=50_000), np.full(30_000, 10), rng.integers(0, 11, size=5_000),
                          np.full(7, 899_999), np.zeros(9, dtype=np.int64)])
    rng.shuffle(idx)
    out = run_unique(wgb, torch, torch.from_numpy(idx.astype(np.int64)).cuda(), first_row)
    check(orc, idx, first_row, *out)


def test_unique_by_owner_large_table_ids(gpu, wgb, orc):
    """Row ids of a 240,000,000-row table (28 key bits), 8 owners, a Zipf-like list."""
    import torch
    rng = np.random.default_rng(6)
    rows, n = 240_000_000, 300_000
    first_row = [int(x) for x in orc.equal_partition_offsets(rows, 8)]
    head = rng.integers(0, 2_000, size=n // 2) * 119_993 % rows        # many repeats of few ids
    idx = np.concatenate([head, rng.integers(0, rows, size=n - n // 2)]).astype(np.int64)
    rng.shuffle(idx)
    idx[:5] = [0, rows - 1, first_row[1], first_row[1] - 1, first_row[7]]
    out = run_unique(wgb, torch, torch.from_numpy(idx).cuda(), first_row)
    check(orc, idx, first_row, *out)


def check_any_order(orc, idx, first_row, unique_ids, inverse, counts, starts):
    """The unordered form: every owner's group holds exactly that owner's distinct ids, in any
    order; every list position finds its own id through `inverse`."""
    rows, n = first_row[-1], idx.shape[0]
    idx64 = idx.astype(np.int64)
    valid = (idx64 >= 0) & (idx64 < rows)
    want = np.unique(idx64[valid])
    want_counts, _, _ = orc.bucket_sort_ids(want, np.asarray(first_row, dtype=np.int64))
    assert np.array_equal(counts, want_counts)
    assert np.array_equal(starts, np.concatenate([[0], np.cumsum(want_counts)[:-1]]))
    for r in range(len(first_row) - 1):
        group = unique_ids[int(starts[r]):int(starts[r] + counts[r])]
        mine = want[(want >= first_row[r]) & (want < first_row[r + 1])]
        assert np.array_equal(np.sort(group), mine), f"group of rank {r}"
    if n:
        inv = inverse[:n]
        assert np.all(inv[~valid] == -1)
        assert np.array_equal(unique_ids[inv[valid]], idx64[valid])


@pytest.mark.parametrize("world", [1, 2, 8, 64])
@pytest.mark.parametrize("n", [0, 1, 257, 4096, 100_003])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_unique_by_owner_any_order(gpu, wgb, orc, world, n, idx_dtype):
    import torch
    rng = np.random.default_rng(world * 31 + n)
    rows = 1_000_003
    first_row = [int(x) for x in orc.equal_partition_offsets(rows, world)]
    idx = rng.integers(0, rows, size=n).astype(idx_dtype)
    if n > 8:
        idx[: n // 3] = idx[n // 3: 2 * (n // 3)]
        idx[rng.integers(0, n, size=n // 10)] = -1
        idx[rng.integers(0, n, size=3)] = rows + 5
    out = run_unique(wgb, torch, torch.from_numpy(idx).cuda(), first_row, "wholegraph_b200_unique_by_owner_any_order")
    check_any_order(orc, idx, first_row, *out)


def test_unique_by_owner_any_order_with_one_id_taking_a_tenth_of_the_list(gpu, wgb, orc):
    """A Zipf-like list over a 240,000,000-row table: one id takes 10 % of 2,000,000 positions, a
    few thousand ids most of the rest; uneven shards."""
    import torch
    rng = np.random.default_rng(8)
    rows, n = 240_000_000, 2_000_000
    first_row = [0, 10, 30_000_000, 30_000_001, 119_999_999, 120_000_000, 200_000_000, 239_999_999, rows]
    head = rng.integers(0, 3_000, size=n) * 79_999 % rows
    idx = np.where(rng.random(n) < 0.7, head, rng.integers(0, rows, size=n)).astype(np.int64)
    idx[rng.random(n) < 0.1] = 123_456_789
    idx[:6] = [0, rows - 1, 9, 10, 30_000_000, 239_999_998]
    out = run_unique(wgb, torch, torch.from_numpy(idx).cuda(), first_row, "wholegraph_b200_unique_by_owner_any_order")
    check_any_order(orc, idx, first_row, *out)
