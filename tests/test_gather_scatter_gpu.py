"""GPU parity of wholegraph_gather / wholegraph_scatter against the CPU oracle, through the C ABI.

The parameter grid follows the reference's gtest grids
(cpp/tests/wholegraph_tensor_ops/wholegraph_gather_tests.cu:271-413,
wholegraph_scatter_tests.cu:281-404): empty request lists, dims 1/11/32/127/128/129/513,
row strides above the dim, storage offsets, every legal dtype pair, int32 and int64 indices,
negative indices.  Everything is compared bit for bit.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FLOATS = [1, 2, 3, 4]   # fp32 fp16 fp64 bf16
INTS = [5, 6, 7, 8]     # int32 int64 int16 int8


def _random_table(rng, orc, rows, cols, dt):
    """Random contents as the numpy carrier dtype of wholegraph dtype `dt`."""
    npdt = orc.np_dtype(dt)
    if dt in (1, 3):
        return rng.uniform(-1, 1, size=(rows, cols)).astype(npdt)
    if dt == 2:
        return rng.uniform(-1, 1, size=(rows, cols)).astype(np.float16)
    if dt == 4:
        return orc.float_to_bf16_bits(rng.uniform(-1, 1, size=(rows, cols)).astype(np.float32))
    info = np.iinfo(npdt)
    return rng.integers(info.min, info.max, size=(rows, cols), dtype=npdt, endpoint=True)


def _to_device(torch, a, dt):
    t = torch.from_numpy(a.view(np.int16) if dt == 4 else a).cuda()
    return t.view(torch.bfloat16) if dt == 4 else t


def _to_host(torch, t, dt):
    if dt == 4:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def _run_gather(gpu, wgb, orc, rng, rows, dim, stride, offset, tab_dt, out_dt, n, idx_np_dtype,
                out_stride=None, negatives=True):
    import torch
    out_stride = out_stride or dim
    storage = _random_table(rng, orc, rows, stride, tab_dt).reshape(-1)
    pad = _random_table(rng, orc, 1, offset + 1, tab_dt).reshape(-1)[:offset]
    storage = np.concatenate([pad, storage])
    idx = rng.integers(0, rows, size=n).astype(idx_np_dtype)
    if negatives and n > 3:
        idx[rng.integers(0, n, size=max(1, n // 16))] = -1
    d_storage = _to_device(torch, storage, tab_dt)
    d_idx = torch.from_numpy(idx).cuda()
    sentinel = np.ascontiguousarray(_random_table(rng, orc, max(n, 1), out_stride, out_dt)[:n])
    d_out = _to_device(torch, sentinel.copy(), out_dt)

    desc = wgb.make_description([rows, dim], wgb.WholeGraphDataType(tab_dt), strides=[stride, 1],
                                storage_offset=offset)
    wt = wgb.make_tensor_from_pointer(d_storage.data_ptr(), desc)
    odesc = wgb.make_description([n, dim], wgb.WholeGraphDataType(out_dt), strides=[out_stride, 1])
    wo = wgb.make_tensor_from_pointer(d_out.data_ptr(), odesc)
    wi = gpu.wrap_torch_tensor(d_idx)
    try:
        wgb.wholegraph_gather_op(wt, wi, wo, wgb.cached_env_fns(), gpu.current_stream_int())
        torch.cuda.synchronize()
    finally:
        for t in (wt, wo, wi):
            wgb.destroy_wholegraph_tensor(t)
    table_view = storage[offset:offset + rows * stride].reshape(rows, stride)[:, :dim]
    want = sentinel.copy()
    orc.gather(table_view, idx, out_dt=out_dt, out=want[:, :dim], table_bf16=(tab_dt == 4))
    got = _to_host(torch, d_out, out_dt)
    assert np.array_equal(got.view(want.dtype), want)


@pytest.mark.parametrize("dim,stride,offset", [(1, 1, 0), (11, 11, 0), (32, 32, 0), (127, 127, 0),
                                               (128, 128, 0), (129, 129, 0), (513, 513, 0),
                                               (128, 130, 2), (11, 12, 0), (32, 33, 1), (64, 72, 8)])
@pytest.mark.parametrize("tab_dt,out_dt", [(1, 1), (1, 2), (1, 4), (2, 2), (2, 1), (4, 4), (4, 1)])
def test_gather_shapes(gpu, wgb, orc, dim, stride, offset, tab_dt, out_dt):
    rng = np.random.default_rng(dim * 1000 + stride * 10 + tab_dt * 3 + out_dt)
    _run_gather(gpu, wgb, orc, rng, 5000, dim, stride, offset, tab_dt, out_dt, 1537, np.int64)


@pytest.mark.parametrize("tab_dt", FLOATS)
@pytest.mark.parametrize("out_dt", FLOATS)
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_gather_float_pairs(gpu, wgb, orc, tab_dt, out_dt, idx_dtype):
    rng = np.random.default_rng(tab_dt * 16 + out_dt)
    for dim in (8, 30, 128):
        _run_gather(gpu, wgb, orc, rng, 3000, dim, dim, 0, tab_dt, out_dt, 777, idx_dtype)


@pytest.mark.parametrize("tab_dt", INTS)
@pytest.mark.parametrize("out_dt", INTS)
def test_gather_int_pairs(gpu, wgb, orc, tab_dt, out_dt):
    rng = np.random.default_rng(tab_dt * 16 + out_dt)
    for dim in (1, 16, 100):
        _run_gather(gpu, wgb, orc, rng, 3000, dim, dim, 0, tab_dt, out_dt, 900, np.int64)


@pytest.mark.parametrize("tab_dt,out_dt,dim", [(1, 2, 128), (1, 4, 128), (1, 1, 128), (2, 2, 128), (4, 4, 128),
                                               (2, 1, 128), (4, 1, 64), (1, 2, 16), (1, 1, 192), (2, 2, 384),
                                               (1, 2, 20), (2, 4, 40), (3, 3, 8), (6, 6, 16), (8, 8, 64)])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_gather_long_lists(gpu, wgb, orc, tab_dt, out_dt, dim, idx_dtype):
    """Request lists long enough for the bulk-copy (shared-memory staged) gather kernel,
    including row sizes at and beyond its limits, which fall back to the register kernel."""
    rng = np.random.default_rng(tab_dt * 7 + out_dt * 3 + dim)
    _run_gather(gpu, wgb, orc, rng, 60000, dim, dim, 0, tab_dt, out_dt, 40001, idx_dtype)
    _run_gather(gpu, wgb, orc, rng, 60000, dim, dim + 8, 8, tab_dt, out_dt, 9000, idx_dtype,
                out_stride=dim + 16)


@pytest.mark.parametrize("n", [0, 1, 31, 32, 33, 255, 257])
def test_gather_list_lengths(gpu, wgb, orc, n):
    rng = np.random.default_rng(n)
    _run_gather(gpu, wgb, orc, rng, 1000, 128, 128, 0, 1, 2, n, np.int64)
    _run_gather(gpu, wgb, orc, rng, 1000, 128, 128, 0, 2, 2, n, np.int32, out_stride=136)


def test_gather_1d_table(gpu, wgb, orc):
    import torch
    rng = np.random.default_rng(5)
    table = rng.integers(-10**12, 10**12, size=20000, dtype=np.int64)
    idx = rng.integers(0, 20000, size=3001).astype(np.int64)
    idx[7] = -1
    d_table, d_idx = torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda()
    d_out = torch.full((3001,), -5, dtype=torch.int64, device="cuda")
    wt = gpu.wrap_torch_tensor(d_table)
    gpu.gather(wt, d_idx, d_out)
    torch.cuda.synchronize()
    wgb.destroy_wholegraph_tensor(wt)
    want = orc.gather(table, idx, out=np.full(3001, -5, dtype=np.int64))
    assert np.array_equal(d_out.cpu().numpy(), want)


def test_gather_rejects_bad_arguments(gpu, wgb):
    import torch
    table = torch.zeros((10, 4), dtype=torch.float32, device="cuda")
    idx = torch.zeros(3, dtype=torch.int64, device="cuda")
    wt = gpu.wrap_torch_tensor(table)
    # float table into an integer output
    with pytest.raises(wgb.WholeGraphError) as e:
        gpu.gather(wt, idx, torch.zeros((3, 4), dtype=torch.int32, device="cuda"))
    assert e.value.code == wgb.ErrorCode.LOGIC_ERROR
    # row count mismatch
    with pytest.raises(wgb.WholeGraphError) as e:
        gpu.gather(wt, idx, torch.zeros((4, 4), dtype=torch.float32, device="cuda"))
    assert e.value.code == wgb.ErrorCode.LOGIC_ERROR
    # 1-D output for a 2-D table
    with pytest.raises(wgb.WholeGraphError) as e:
        gpu.gather(wt, idx, torch.zeros(3, dtype=torch.float32, device="cuda"))
    assert e.value.code == wgb.ErrorCode.INVALID_INPUT
    wgb.destroy_wholegraph_tensor(wt)


@pytest.mark.parametrize("in_dt,tab_dt", [(1, 1), (2, 1), (1, 2), (4, 1), (1, 4), (3, 2), (2, 2),
                                          (5, 6), (8, 5), (6, 7)])
@pytest.mark.parametrize("dim,stride,offset", [(1, 1, 0), (11, 12, 0), (128, 128, 0), (129, 131, 2),
                                               (513, 513, 0)])
def test_scatter(gpu, wgb, orc, in_dt, tab_dt, dim, stride, offset):
    import torch
    rng = np.random.default_rng(in_dt * 100 + tab_dt * 10 + dim)
    rows, n = 4000, 1111
    storage = _random_table(rng, orc, rows + 1, stride, tab_dt).reshape(-1)
    idx = rng.permutation(rows)[:n].astype(np.int64)  # unique: duplicate writers race
    idx[5] = -1
    inp = _random_table(rng, orc, n, dim, in_dt)
    d_storage = _to_device(torch, storage.copy(), tab_dt)
    d_in, d_idx = _to_device(torch, inp, in_dt), torch.from_numpy(idx).cuda()
    desc = wgb.make_description([rows, dim], wgb.WholeGraphDataType(tab_dt), strides=[stride, 1],
                                storage_offset=offset)
    wt = wgb.make_tensor_from_pointer(d_storage.data_ptr(), desc)
    gpu.scatter(d_in, d_idx, wt)
    torch.cuda.synchronize()
    wgb.destroy_wholegraph_tensor(wt)
    want = storage.copy()
    view = want[offset:offset + rows * stride].reshape(rows, stride)[:, :dim]
    orc.scatter(inp, idx, view, rows_bf16=(in_dt == 4), table_bf16=(tab_dt == 4))
    got = _to_host(torch, d_storage, tab_dt)
    assert np.array_equal(got.view(want.dtype), want)


def test_config1_gather_then_scatter(gpu, wgb, orc):
    """1,000,000 x 128 fp32 table (seed 0), 65,536 int64 ids (seed 1), gather to fp32, then
    scatter 65,536 unique-id fp32 rows (seed 2); bit-exact."""
    import torch
    rows, dim, n = 1_000_000, 128, 65_536
    table = np.random.default_rng(0).uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    idx = np.random.default_rng(1).integers(0, rows, size=n, dtype=np.int64)
    d_table, d_idx = torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda()
    wt = gpu.wrap_torch_tensor(d_table)
    out = torch.empty((n, dim), dtype=torch.float32, device="cuda")
    gpu.gather(wt, d_idx, out)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), orc.gather(table, idx, threads=8))
    rng2 = np.random.default_rng(2)
    uniq = rng2.permutation(rows)[:n].astype(np.int64)
    new_rows = rng2.uniform(-1, 1, size=(n, dim)).astype(np.float32)
    gpu.scatter(torch.from_numpy(new_rows).cuda(), torch.from_numpy(uniq).cuda(), wt)
    torch.cuda.synchronize()
    wgb.destroy_wholegraph_tensor(wt)
    orc.scatter(new_rows, uniq, table, threads=8)
    assert np.array_equal(d_table.cpu().numpy(), table)


def test_config2_cast_gather_properties(gpu, wgb, orc):
    """10,000,000 x 128 fp32 table, 1,048,576 ids with replacement, gather with fused cast to
    fp16 and bf16, then scatter of 1,048,576 unique-id fp16 rows.  Full-size run checked against
    the oracle on a sample of rows and through size-independent properties: equal ids give
    equal rows, the cast equals torch's round-to-nearest-even cast of the same rows, and a
    scatter followed by a gather of the same ids returns the scattered rows."""
    import torch
    rows, dim, n = 10_000_000, 128, 1_048_576
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.empty((rows, dim), dtype=torch.float32, device="cuda").uniform_(-1, 1, generator=g)
    idx = torch.randint(0, rows, (n,), generator=torch.Generator(device="cuda").manual_seed(1),
                        device="cuda", dtype=torch.int64)
    wt = gpu.wrap_torch_tensor(table)
    for dt, wg in ((torch.float16, 2), (torch.bfloat16, 4)):
        out = torch.empty((n, dim), dtype=dt, device="cuda")
        gpu.gather(wt, idx, out)
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), table[idx].to(dt).view(torch.int16))
        sample = torch.arange(0, n, 997, device="cuda")
        want = orc.gather(table[idx[sample]].cpu().numpy(), np.arange(sample.numel()), out_dt=wg)
        assert np.array_equal(out[sample].view(torch.int16).cpu().numpy().view(want.dtype), want)
    uniq = torch.randperm(rows, generator=torch.Generator(device="cuda").manual_seed(2), device="cuda")[:n]
    new_rows = torch.empty((n, dim), dtype=torch.float16, device="cuda").uniform_(-1, 1)
    gpu.scatter(new_rows, uniq, wt)
    back = torch.empty((n, dim), dtype=torch.float16, device="cuda")
    gpu.gather(wt, uniq, back)
    torch.cuda.synchronize()
    assert torch.equal(back, new_rows)  # fp16 -> fp32 -> fp16 is the identity
    wgb.destroy_wholegraph_tensor(wt)


def test_wholememory_spelling_gathers_and_scatters(gpu, wgb, orc):
    """wholememory_gather / wholememory_scatter - the names the C API had before the reference's
    rename, still used by its torch extension (torch_cpp_ext/torch_utils.cpp:11-181) - are exported
    and do the same work: fp32 table, fp16 output, then fp16 rows scattered back."""
    import ctypes as C
    import torch
    lib = wgb.lib()
    for name in ("wholememory_gather", "wholememory_scatter"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = C.c_int, [C.c_void_p] * 3 + [C.POINTER(wgb.EnvFns), C.c_void_p, C.c_int]
    rng = np.random.default_rng(21)
    rows, dim, n = 30_000, 128, 5_000
    table = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    idx = rng.integers(0, rows, size=n).astype(np.int64)
    idx[::41] = -1
    d_table, d_idx = torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda()
    out = torch.zeros((n, dim), dtype=torch.float16, device="cuda")
    wt, wi, wo = gpu.wrap_torch_tensor(d_table), gpu.wrap_torch_tensor(d_idx), gpu.wrap_torch_tensor(out)
    stream = C.c_void_p(gpu.current_stream_int())
    assert lib.wholememory_gather(wt, wi, wo, wgb.cached_env_fns(), stream, -1) == 0
    torch.cuda.synchronize()
    want = orc.gather(table, idx, out_dt=orc.DT_HALF, out=np.zeros((n, dim), dtype=np.float16))
    assert np.array_equal(out.cpu().numpy().view(np.int16), want.view(np.int16))
    perm = rng.permutation(rows)[:n].astype(np.int64)
    rows_in = rng.uniform(-1, 1, size=(n, dim)).astype(np.float16)
    d_rows, d_perm = torch.from_numpy(rows_in).cuda(), torch.from_numpy(perm).cuda()
    wr, wp = gpu.wrap_torch_tensor(d_rows), gpu.wrap_torch_tensor(d_perm)
    assert lib.wholememory_scatter(wr, wp, wt, wgb.cached_env_fns(), stream, -1) == 0
    torch.cuda.synchronize()
    want_table = table.copy()
    orc.scatter(rows_in, perm, want_table)
    assert np.array_equal(d_table.cpu().numpy(), want_table)
    for w in (wt, wi, wo, wr, wp):
        wgb.destroy_wholegraph_tensor(w)


@pytest.mark.parametrize("mem_name", ["MtContinuous", "MtDistributed"])
@pytest.mark.parametrize("tab_dt,out_dt", [(1, 2), (2, 2), (6, 6)])
def test_host_resident_tables(gpu, wgb, orc, mem_name, tab_dt, out_dt):
    """Tables in pinned host memory (CONTINUOUS / HOST and DISTRIBUTED / HOST handles, reference:
    cpp/src/wholegraph/memory_handle.cpp:503-546): the same kernels read and write them through
    their device-visible addresses; results must equal the oracle's, as for device tables
    (reference grid: wholegraph_gather_tests.cu:271-413 runs every case for HOST as well)."""
    import torch
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    rng = np.random.default_rng(tab_dt * 10 + out_dt)
    rows, dim, n = 20_000, 96, 7_000
    table_np = _random_table(rng, orc, rows, dim, tab_dt)
    t = wgb.create_wholegraph_tensor(wgb.make_description([rows, dim], DT(tab_dt)), comm, getattr(MT, mem_name), ML.MlHost)
    gpu.write_local_shard(t, _to_device(torch, table_np, tab_dt).contiguous())
    idx = rng.integers(0, rows, size=n).astype(np.int64)
    idx[::53] = -1
    sentinel = _random_table(rng, orc, n, dim, out_dt)
    d_out = _to_device(torch, sentinel.copy(), out_dt)
    gpu.gather(t, torch.from_numpy(idx).cuda(), d_out)
    torch.cuda.synchronize()
    want = sentinel.copy()
    orc.gather(table_np, idx, out_dt=out_dt, out=want, table_bf16=(tab_dt == 4))
    assert np.array_equal(_to_host(torch, d_out, out_dt).view(want.dtype), want)
    # scatter back into the host table at unique ids and read it through a gather of all rows
    perm = rng.permutation(rows)[:n].astype(np.int64)
    rows_in = _random_table(rng, orc, n, dim, out_dt)
    gpu.scatter(_to_device(torch, rows_in, out_dt), torch.from_numpy(perm).cuda(), t)
    back = _to_device(torch, np.zeros_like(table_np), tab_dt)
    gpu.gather(t, torch.arange(rows, device="cuda", dtype=torch.int64), back)
    torch.cuda.synchronize()
    want_table = table_np.copy()
    orc.scatter(rows_in, perm, want_table, rows_bf16=(out_dt == 4), table_bf16=(tab_dt == 4))
    assert np.array_equal(_to_host(torch, back, tab_dt).view(want_table.dtype), want_table)
    wgb.destroy_wholegraph_tensor(t)
    wgb.destroy_communicator(comm)


@pytest.mark.parametrize("mem_name", ["MtContinuous", "MtDistributed", "MtChunked"])
def test_gather_from_a_handle_with_raw_pointers(gpu, wgb, orc, mem_name):
    """The form in which NCCL-mode neighbour sampling calls the gather (reference:
    cpp/src/wholegraph_ops/unweighted_sample_without_replacement_nccl_func.cuh:236, :364): a memory
    handle, descriptors and raw device pointers; an int64 CSR row-pointer array gathered at
    [v, v + 1] pairs, then column ids gathered at edge positions (int32 columns, int64 output)."""
    import ctypes as C
    import torch
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    lib = wgb.lib()
    comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    rng = np.random.default_rng(31)
    nodes, centers = 40_000, 3_000
    degree = rng.integers(0, 12, size=nodes)
    row_ptr = np.concatenate([[0], np.cumsum(degree)]).astype(np.int64)
    col = rng.integers(0, nodes, size=int(row_ptr[-1])).astype(np.int32)

    def handle_with(values, dt):
        t = wgb.create_wholegraph_tensor(wgb.make_description([len(values)], dt), comm, getattr(MT, mem_name), ML.MlDevice)
        gpu.write_local_shard(t, torch.from_numpy(values).cuda())
        return t, C.c_void_p(lib.wholegraph_tensor_get_memory_handle(t))

    t_row, h_row = handle_with(row_ptr, DT.DtInt64)
    t_col, h_col = handle_with(col, DT.DtInt)
    env, stream = wgb.cached_env_fns(), C.c_void_p(gpu.current_stream_int())
    v = rng.integers(0, nodes, size=centers).astype(np.int64)
    pairs = np.concatenate([[-7, -7, -7], v, v + 1]).astype(np.int64)        # three elements of storage offset
    d_pairs = torch.from_numpy(pairs).cuda()
    out = torch.full((2 * centers + 5,), -1, dtype=torch.int64, device="cuda")
    tab = wgb.MatrixDescription((len(row_ptr), 1), 1, 0, int(DT.DtInt64))
    idd = wgb.ArrayDescription(2 * centers, 3, int(DT.DtInt64))
    od = wgb.MatrixDescription((2 * centers, 1), 1, 5, int(DT.DtInt64))
    rc = lib.wholegraph_b200_gather_from_handle(h_row, C.byref(tab), C.c_void_p(d_pairs.data_ptr()), C.byref(idd),
                                                C.c_void_p(out.data_ptr()), C.byref(od), env, stream, -1)
    assert rc == 0
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.all(got[:5] == -1)
    assert np.array_equal(got[5:5 + centers], row_ptr[v]) and np.array_equal(got[5 + centers:], row_ptr[v + 1])
    # column ids at sampled edge positions, int32 ids widened to int64 by the gather's cast
    has_edges = v[degree[v] > 0]
    edges = (row_ptr[has_edges] + rng.integers(0, 1 << 30, size=len(has_edges)) % degree[has_edges]).astype(np.int64)
    d_edges = torch.from_numpy(edges).cuda()
    dst = torch.zeros(len(edges), dtype=torch.int64, device="cuda")
    tab = wgb.MatrixDescription((len(col), 1), 1, 0, int(DT.DtInt))
    idd = wgb.ArrayDescription(len(edges), 0, int(DT.DtInt64))
    od = wgb.MatrixDescription((len(edges), 1), 1, 0, int(DT.DtInt64))
    rc = lib.wholegraph_b200_gather_from_handle(h_col, C.byref(tab), C.c_void_p(d_edges.data_ptr()), C.byref(idd),
                                                C.c_void_p(dst.data_ptr()), C.byref(od), env, stream, -1)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), col[edges].astype(np.int64))
    # argument checks
    bad = wgb.MatrixDescription((len(edges), 1), 1, 0, int(DT.DtFloat))
    assert lib.wholegraph_b200_gather_from_handle(h_col, C.byref(tab), C.c_void_p(d_edges.data_ptr()), C.byref(idd),
                                                  C.c_void_p(dst.data_ptr()), C.byref(bad), env, stream, -1) == int(wgb.ErrorCode.LOGIC_ERROR)
    assert lib.wholegraph_b200_gather_from_handle(None, C.byref(tab), None, C.byref(idd), None, C.byref(od), env, stream, -1) \
        == int(wgb.ErrorCode.INVALID_INPUT)
    wgb.destroy_wholegraph_tensor(t_row)
    wgb.destroy_wholegraph_tensor(t_col)
    wgb.destroy_communicator(comm)


@pytest.mark.parametrize("switches", [{}, {"WG_SERVE_BULK": "0"}, {"WG_SYNC_FREE": "0"}, {"WG_PEER_EXCHANGE": "0"},
                                      {"WG_GATHER_DEDUP": "0"},
                                      {"WG_GATHER_DEDUP": "0", "WG_PEER_EXCHANGE": "0", "WG_EXCHANGE_CHUNKS": "3"}],
                         ids=["sync-free", "sync-free-register-kernel", "host-counts", "nccl-rows", "keep-duplicates",
                              "keep-duplicates-chunked"])
@pytest.mark.parametrize("tab_dt,out_dt,dim", [(4, 4, 128), (2, 1, 33), (1, 2, 64), (6, 6, 5)])
def test_distributed_exchange_code_on_one_rank(gpu, wgb, orc, monkeypatch, switches, tab_dt, out_dt, dim):
    """WG_SINGLE_RANK_EXCHANGE=1 makes a one-rank communicator run the exchange code of a DISTRIBUTED
    gather and scatter - de-duplication, request header and ids in the exchange arena, the owner's
    serve kernel, the expansion, or the routed / chunked variants the other switches select - with
    itself as its only peer, so that this code is checked against the oracle on one GPU as well.
    (The reference runs its distributed path on one rank the same way: on a one-GPU box its gtests
    degenerate to world size 1, cpp/tests/wholegraph_tensor_ops/wholegraph_gather_tests.cu:126-269.)"""
    import torch
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    monkeypatch.setenv("WG_SINGLE_RANK_EXCHANGE", "1")
    for k, v in switches.items():
        monkeypatch.setenv(k, v)
    comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)      # reads the switches
    rng = np.random.default_rng(tab_dt * 100 + out_dt + dim)
    rows = 30_011
    table_np = _random_table(rng, orc, rows, dim, tab_dt)
    t = wgb.create_wholegraph_tensor(wgb.make_description([rows, dim], DT(tab_dt)), comm, MT.MtDistributed, ML.MlDevice)
    gpu.write_local_shard(t, _to_device(torch, table_np, tab_dt).contiguous())
    launches = wgb.lib().wholegraph_b200_kernel_launch_count()
    for n in (12_345, 0, 1, 40_000):
        idx = rng.integers(0, rows, size=n).astype(np.int64)
        if n > 10:
            idx[: n // 3] = idx[n // 3: 2 * (n // 3)]            # duplicates
            idx[::37] = -1
            idx[5] = rows + 3                                    # nobody's row: left untouched
        sentinel = _random_table(rng, orc, max(n, 1), dim, out_dt)[:n]
        d_out = _to_device(torch, sentinel.copy(), out_dt)
        gpu.gather(t, torch.from_numpy(idx).cuda(), d_out)
        torch.cuda.synchronize()
        want = sentinel.copy()
        orc.gather(table_np, np.where(idx >= rows, -1, idx), out_dt=out_dt, out=want, table_bf16=(tab_dt == 4))
        assert np.array_equal(_to_host(torch, d_out, out_dt).view(want.dtype), want), f"n={n}"
    if not switches:
        assert wgb.lib().wholegraph_b200_kernel_launch_count() - launches >= 3 * 6   # not the one-kernel shortcut
    # scatter through the routed exchange, then read back
    n = 9_000
    perm = rng.permutation(rows)[:n].astype(np.int64)
    rows_in = _random_table(rng, orc, n, dim, out_dt)
    gpu.scatter(_to_device(torch, rows_in, out_dt), torch.from_numpy(perm).cuda(), t)
    back = _to_device(torch, np.zeros_like(table_np), tab_dt)
    gpu.gather(t, torch.arange(rows, device="cuda", dtype=torch.int64), back)
    torch.cuda.synchronize()
    want_table = table_np.copy()
    orc.scatter(rows_in, perm, want_table, rows_bf16=(out_dt == 4), table_bf16=(tab_dt == 4))
    assert np.array_equal(_to_host(torch, back, tab_dt).view(want_table.dtype), want_table)
    wgb.destroy_wholegraph_tensor(t)
    wgb.destroy_communicator(comm)


@pytest.mark.parametrize("dim", [64, 128, 136, 512, 4096, 4104])
def test_distributed_gather_with_bulk_copies_over_row_sizes(gpu, wgb, orc, monkeypatch, dim):
    """The owner-side kernel of the default path stages tiles of rows in shared memory with bulk
    asynchronous copies and sends each tile with one bulk store.  bf16 rows of 128 bytes to 8 KiB
    (tiles of 32 down to 1 rows) and two widths the bulk form does not take (272 bytes is a
    multiple of 16 but 8208 exceeds a buffer: the register kernel serves those), a list with
    repeats, skipped positions and a group that ends inside a tile; against the oracle, bit for bit."""
    import torch
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    monkeypatch.setenv("WG_SINGLE_RANK_EXCHANGE", "1")
    comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    rng = np.random.default_rng(dim)
    rows = 20_011 if dim <= 512 else 3_001
    table_np = _random_table(rng, orc, rows, dim, 4)
    t = wgb.create_wholegraph_tensor(wgb.make_description([rows, dim], DT(4)), comm, MT.MtDistributed, ML.MlDevice)
    gpu.write_local_shard(t, _to_device(torch, table_np, 4).contiguous())
    for n in (1, 33, 2 * rows + 7):
        idx = rng.integers(0, rows, size=n).astype(np.int64)
        if n > 10:
            idx[::41] = -1
        sentinel = _random_table(rng, orc, n, dim, 4)
        d_out = _to_device(torch, sentinel.copy(), 4)
        gpu.gather(t, torch.from_numpy(idx).cuda(), d_out)
        torch.cuda.synchronize()
        want = sentinel.copy()
        orc.gather(table_np, idx, out_dt=4, out=want, table_bf16=True)
        assert np.array_equal(_to_host(torch, d_out, 4).view(want.dtype), want), f"n={n}"
    wgb.destroy_wholegraph_tensor(t)
    wgb.destroy_communicator(comm)
