"""GPU tests of graph_append_unique and csr_add_self_loop through the C ABI against the oracle and
against the properties the reference's own tests check
(cpp/tests/graph_ops/append_unique_tests.cu, csr_add_self_loop_tests.cu): targets first and
unchanged, every other neighbour exactly once, mapping consistent with the list; self loop first in
every row.  The order of the appended neighbours is ascending here (the reference's is the order
of its hash table), so the comparison with the oracle is exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _append_unique(gpu, wgb, torch, targets, neighbors, want_mapping=True):
    d_t, d_n = torch.from_numpy(targets).cuda(), torch.from_numpy(neighbors).cuda()
    d_map = torch.full((max(len(neighbors), 1),), -7, dtype=torch.int32, device="cuda")[:len(neighbors)]
    wt, wn = gpu.wrap_torch_tensor(d_t), gpu.wrap_torch_tensor(d_n)
    wm = gpu.wrap_torch_tensor(d_map) if want_mapping else None
    slot = wgb.OutputSlot()
    wgb.append_unique(wt, wn, slot, wm, wgb.cached_env_fns(), gpu.current_stream_int())
    torch.cuda.synchronize()
    n_unique = slot.description.sizes[0]
    assert slot.description.dim == 1 and slot.description.dtype == gpu.TORCH_TO_WG[d_t.dtype]
    unique = gpu.view_device_memory(slot.pointer, [n_unique], d_t.dtype, [1]).clone().cpu().numpy() if n_unique else \
        np.zeros(0, dtype=targets.dtype)
    wgb.release_output(slot)
    assert slot.pointer is None
    for w in (wt, wn, wm):
        if w is not None:
            wgb.destroy_wholegraph_tensor(w)
    return unique, d_map.cpu().numpy()


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
@pytest.mark.parametrize("t_count,n_count,span", [(1, 1, 4), (10, 100, 50), (513, 4099, 3000), (1000, 100_003, 40_000),
                                                  (0, 77, 30), (64, 0, 100)])
def test_append_unique_matches_the_oracle(gpu, wgb, orc, dtype, t_count, n_count, span):
    import torch
    rng = np.random.default_rng(t_count * 31 + n_count)
    base = 5_000_000_000 if dtype == np.int64 else 7
    targets = (rng.permutation(span)[:t_count] + base).astype(dtype)            # distinct, unordered
    neighbors = (rng.integers(0, span, size=n_count) + base).astype(dtype)      # duplicates, some are targets
    unique, mapping = _append_unique(gpu, wgb, torch, targets, neighbors)
    want_unique, want_mapping = orc.append_unique(targets, neighbors)
    assert np.array_equal(unique, want_unique)
    assert np.array_equal(mapping, want_mapping)
    # the reference's properties, independent of the order of the appended part
    assert np.array_equal(unique[:t_count], targets)
    assert len(np.unique(unique)) == len(unique)
    assert set(unique.tolist()) == set(targets.tolist()) | set(neighbors.tolist())
    if n_count:
        assert np.array_equal(unique[mapping], neighbors)


def test_append_unique_without_mapping_and_with_repeated_targets(gpu, wgb, orc):
    import torch
    targets = np.array([9, 3, 9, 5], dtype=np.int64)          # a repeated target keeps its first position
    neighbors = np.array([5, 9, 1, 1, 3, 12], dtype=np.int64)
    unique, _ = _append_unique(gpu, wgb, torch, targets, neighbors, want_mapping=False)
    assert unique.tolist() == [9, 3, 9, 5, 1, 12]
    unique, mapping = _append_unique(gpu, wgb, torch, targets, neighbors)
    assert mapping.tolist() == [3, 0, 4, 4, 1, 5]
    assert (unique.tolist(), mapping.tolist()) == tuple(x.tolist() for x in orc.append_unique(targets, neighbors))


def test_append_unique_refuses_mixed_id_types(gpu, wgb):
    import torch
    wt = gpu.wrap_torch_tensor(torch.zeros(4, dtype=torch.int32, device="cuda"))
    wn = gpu.wrap_torch_tensor(torch.zeros(4, dtype=torch.int64, device="cuda"))
    slot = wgb.OutputSlot()
    with pytest.raises(wgb.WholeGraphError):
        wgb.append_unique(wt, wn, slot, None, wgb.cached_env_fns(), 0)
    wgb.destroy_wholegraph_tensor(wt)
    wgb.destroy_wholegraph_tensor(wn)


@pytest.mark.parametrize("rows,max_degree", [(1, 0), (1, 5), (33, 3), (1000, 40), (20_000, 100)])
def test_csr_add_self_loop_matches_the_oracle(gpu, wgb, orc, rows, max_degree):
    import torch
    rng = np.random.default_rng(rows + max_degree)
    degree = rng.integers(0, max_degree + 1, size=rows)
    row_ptr = np.concatenate([[0], np.cumsum(degree)]).astype(np.int32)
    col = rng.integers(0, rows, size=int(row_ptr[-1])).astype(np.int32)
    d_rp, d_col = torch.from_numpy(row_ptr).cuda(), torch.from_numpy(col).cuda()
    d_orp = torch.full((rows + 1,), -1, dtype=torch.int32, device="cuda")
    d_ocol = torch.full((len(col) + rows,), -1, dtype=torch.int32, device="cuda")
    ws = [gpu.wrap_torch_tensor(t) for t in (d_rp, d_col, d_orp, d_ocol)]
    wgb.add_csr_self_loop(*ws, gpu.current_stream_int())
    torch.cuda.synchronize()
    want_ptr, want_col = orc.csr_add_self_loop(row_ptr, col)
    assert np.array_equal(d_orp.cpu().numpy(), want_ptr)
    assert np.array_equal(d_ocol.cpu().numpy(), want_col)
    for w in ws:
        wgb.destroy_wholegraph_tensor(w)


def test_csr_add_self_loop_refuses_wrong_types_and_small_outputs(gpu, wgb):
    import torch
    rp = torch.tensor([0, 2, 3], dtype=torch.int32, device="cuda")
    col = torch.tensor([1, 0, 1], dtype=torch.int32, device="cuda")
    good_rp, good_col = torch.zeros(3, dtype=torch.int32, device="cuda"), torch.zeros(5, dtype=torch.int32, device="cuda")
    bad = [(rp.long(), col, good_rp, good_col), (rp, col, good_rp, good_col.long()),
           (rp, col, good_rp[:2], good_col), (rp, col, good_rp, good_col[:4])]
    for tensors in bad:
        ws = [gpu.wrap_torch_tensor(t.contiguous()) for t in tensors]
        with pytest.raises(wgb.WholeGraphError):
            wgb.add_csr_self_loop(*ws, 0)
        for w in ws:
            wgb.destroy_wholegraph_tensor(w)
