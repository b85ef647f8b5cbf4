"""GPU tests of the cached embedding path through the C ABI: forward gather through a
set-associative cache with LFU updates, write-back, drop, and training through the cache.

The reference tests the same properties
(cpp/tests/wholegraph_tensor_ops/wholegraph_embedding_tests.cu, cached cases of
wholegraph_embedding_gradient_apply_tests.cu:798-1007): a cached embedding must return exactly
what the uncached table holds, whatever the cache keeps, and after a write-back the table must
hold what an uncached run would have produced.  The cache policy itself (which rows get the 32
lines of a set) is checked against the oracle's host model of the rule this library states: exact
access counts, highest counts cached, cached rows win ties, then lower row numbers."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

VALID, MODIFIED, ROW_MASK = 1 << 14, 1 << 15, (1 << 14) - 1


@pytest.fixture(scope="module")
def comm(gpu, wgb):
    c = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    yield c
    wgb.destroy_communicator(c)


def _zipf_like(rng, rows, n):
    """Skewed ids: a hot tenth of the table takes most accesses."""
    hot = rng.integers(0, max(rows // 10, 1), size=n)
    cold = rng.integers(0, rows, size=n)
    return np.where(rng.random(n) < 0.8, hot, cold)


def _make(gpu, wgb, comm, rows, dim, torch_dtype, ratio, mem_type=None, cache_type=None, table_location=None):
    MT, ML, AT, DT = (wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphAccessType,
                      wgb.WholeGraphDataType)
    mem_type = mem_type or MT.MtContinuous
    cache_type = cache_type or MT.MtContinuous
    policy = wgb.create_cache_policy(comm, cache_type, ML.MlDevice, AT.AtReadWrite, ratio)
    emb = wgb.create_embedding(wgb.make_description([rows, dim], DT(gpu.TORCH_TO_WG[torch_dtype])), comm,
                               mem_type, table_location or ML.MlDevice, cache_policy=policy)
    return emb, policy


def _read_tensor(gpu, torch, t, rows, cols, dtype):
    ids = torch.arange(rows, device="cuda", dtype=torch.int64)
    out = torch.empty((rows, cols), dtype=dtype, device="cuda")
    gpu.gather(t, ids, out)
    torch.cuda.synchronize()
    return out


def _forward(gpu, wgb, torch, emb, ids_np, dim, dtype, adjust):
    d_ids = torch.from_numpy(ids_np).cuda()
    out = torch.empty((len(ids_np), dim), dtype=dtype, device="cuda")
    wi, wo = gpu.wrap_torch_tensor(d_ids), gpu.wrap_torch_tensor(out)
    wgb.EmbeddingGatherForward(emb, wi, wo, adjust, wgb.cached_env_fns(), gpu.current_stream_int())
    torch.cuda.synchronize()
    wgb.destroy_wholegraph_tensor(wi)
    wgb.destroy_wholegraph_tensor(wo)
    return out


@pytest.mark.parametrize("dtype_name,dim", [("f32", 32), ("f32", 13), ("f16", 64), ("bf16", 100)])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_cached_gather_returns_the_table_and_follows_the_policy(gpu, wgb, orc, comm, dtype_name, dim, idx_dtype):
    import torch
    dtype = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dtype_name]
    rows, ratio = 5000, 0.25                       # coverage 128 -> 40 sets of 32 lines, 5120 rows
    rng = np.random.default_rng(dim * 7 + idx_dtype().itemsize)
    emb, policy = _make(gpu, wgb, comm, rows, dim, dtype, ratio)
    table = wgb.embedding_tensor(emb)
    tags_t, lfu_t, lines_t, coverage = wgb.embedding_cache_tensors(emb)
    assert coverage == 128
    padded_rows = -(-rows // coverage) * coverage
    init = torch.from_numpy(rng.uniform(-1, 1, size=(padded_rows, dim)).astype(np.float32)).cuda().to(dtype)
    gpu.scatter(init, torch.arange(padded_rows, device="cuda", dtype=torch.int64), table)
    torch.cuda.synchronize()
    model = orc.CachePolicyModel(padded_rows, coverage)
    sets = padded_rows // coverage

    for step in range(6):
        ids = _zipf_like(rng, rows, 3000).astype(idx_dtype)
        adjust = step != 3                          # one step only reads
        out = _forward(gpu, wgb, torch, emb, ids, dim, dtype, adjust)
        assert torch.equal(out, init[torch.from_numpy(ids.astype(np.int64)).cuda()]), f"step {step}"
        if adjust:
            model.update(ids.astype(np.int64))
        tags = _read_tensor(gpu, torch, tags_t, sets, 32, torch.int16).cpu().numpy().view(np.uint16)
        for s in range(sets):
            got = {int(t & ROW_MASK): line for line, t in enumerate(tags[s]) if t & VALID}
            assert got == model.cached.get(s, {}), f"step {step} set {s}"
        assert not (tags & MODIFIED).any()
        # every valid line holds its row
        esz = init.element_size()
        pad = -(-dim // (16 // esz)) * (16 // esz)
        lines = _read_tensor(gpu, torch, lines_t, sets * 32, pad, dtype)
        s_idx, l_idx = np.nonzero(tags & VALID)
        src_rows = s_idx * coverage + (tags[s_idx, l_idx] & ROW_MASK)
        assert torch.equal(lines[torch.from_numpy(s_idx * 32 + l_idx).cuda(), :dim],
                           init[torch.from_numpy(src_rows.astype(np.int64)).cuda()])
    # hits must have happened: the hot rows are cached
    assert sum(len(v) for v in model.cached.values()) > 32
    wgb.embedding_drop_all_cache(emb)
    tags = _read_tensor(gpu, torch, tags_t, sets, 32, torch.int16).cpu().numpy()
    assert not tags.any()
    ids = _zipf_like(rng, rows, 500).astype(idx_dtype)
    out = _forward(gpu, wgb, torch, emb, ids, dim, dtype, False)
    assert torch.equal(out, init[torch.from_numpy(ids.astype(np.int64)).cuda()])
    wgb.destroy_embedding(emb)
    wgb.destroy_cache_policy(policy)


def test_cache_ratio_bounds_and_coverage(gpu, wgb, comm):
    import torch
    MT, ML, AT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphAccessType
    p = C.c_void_p()
    for bad in (1.5, 1.0 / 1024):
        rc = wgb.lib().wholegraph_create_embedding_cache_policy(C.byref(p), comm, int(MT.MtContinuous),
                                                                int(ML.MlDevice), int(AT.AtReadWrite), bad)
        assert rc == 7                               # WHOLEGRAPH_INVALID_VALUE
    for ratio, want in ((1.0, 32), (0.5, 64), (0.1, 320), (1.0 / 512, 16384)):
        emb, policy = _make(gpu, wgb, comm, 100, 8, torch.float32, ratio)
        assert wgb.embedding_cache_tensors(emb)[3] == want
        d = wgb.lib().wholegraph_tensor_get_tensor_description(wgb.embedding_tensor(emb)).contents
        assert d.sizes[0] == -(-100 // want) * want  # rows padded to whole sets
        wgb.destroy_embedding(emb)
        wgb.destroy_cache_policy(policy)


def test_a_full_cache_serves_every_row_from_its_lines(gpu, wgb, comm):
    """ratio 1: every row has a line, so after one pass over all ids every later gather hits, and
    overwriting the table behind the cache must not change what a cached gather returns."""
    import torch
    rows, dim = 1024, 16
    emb, policy = _make(gpu, wgb, comm, rows, dim, torch.float32, 1.0)
    table = wgb.embedding_tensor(emb)
    all_ids = torch.arange(rows, device="cuda", dtype=torch.int64)
    init = torch.arange(rows * dim, device="cuda", dtype=torch.float32).reshape(rows, dim)
    gpu.scatter(init, all_ids, table)
    _forward(gpu, wgb, torch, emb, np.arange(rows, dtype=np.int64), dim, torch.float32, True)
    gpu.scatter(torch.zeros_like(init), all_ids, table)          # behind the cache's back
    torch.cuda.synchronize()
    out = _forward(gpu, wgb, torch, emb, np.arange(rows, dtype=np.int64)[::-1].copy(), dim, torch.float32, False)
    assert torch.equal(out, init.flip(0))
    # nothing is modified, so a write-back leaves the zeros in the table
    wgb.embedding_writeback_all_cache(emb)
    assert not _read_tensor(gpu, torch, table, rows, dim, torch.float32).any()
    wgb.destroy_embedding(emb)
    wgb.destroy_cache_policy(policy)


@pytest.mark.parametrize("opt_name,params", [("sgd", {"weight_decay": 0.1}), ("adam", {}),
                                             ("adagrad", {}), ("rmsprop", {"alpha": 0.9})])
@pytest.mark.parametrize("table_dtype,dim", [("f32", 32), ("f32", 129), ("bf16", 64)])
def test_training_through_the_cache_matches_the_oracle(gpu, wgb, orc, comm, opt_name, params, table_dtype, dim):
    from test_optimizer_gpu import _run
    MT = wgb.WholeGraphMemoryType
    _run(gpu, wgb, orc, comm, opt_name, rows=3000, dim=dim, table_dtype=table_dtype, idx_dtype=np.int64,
         steps=5, n=2000, params=params, mem_type=MT.MtContinuous, cache_ratio=0.125)


def test_cached_gather_into_an_output_view_with_a_storage_offset(gpu, wgb, comm):
    """The output may be a strided view that starts some elements into its storage: only the viewed
    elements are written."""
    import torch
    rows, dim, n, offset, stride = 1024, 16, 300, 40, 24
    emb, policy = _make(gpu, wgb, comm, rows, dim, torch.float32, 0.5)
    table = wgb.embedding_tensor(emb)
    init = torch.arange(rows * dim, device="cuda", dtype=torch.float32).reshape(rows, dim)
    gpu.scatter(init, torch.arange(rows, device="cuda", dtype=torch.int64), table)
    ids = torch.randint(0, rows, (n,), device="cuda", dtype=torch.int64)
    storage = torch.empty(offset + n * stride, device="cuda", dtype=torch.float32)
    odesc = wgb.make_description([n, dim], wgb.WholeGraphDataType.DtFloat, strides=[stride, 1], storage_offset=offset)
    wo = wgb.make_tensor_from_pointer(storage.data_ptr(), odesc)
    wi = gpu.wrap_torch_tensor(ids)
    for adjust in (True, False, True):
        storage.fill_(-1.0)
        wgb.EmbeddingGatherForward(emb, wi, wo, adjust, wgb.cached_env_fns(), gpu.current_stream_int())
        torch.cuda.synchronize()
        got = storage[offset:].reshape(n, stride)
        assert torch.equal(got[:, :dim], init[ids])
        assert bool((got[:, dim:] == -1.0).all()) and bool((storage[:offset] == -1.0).all())
    wgb.destroy_wholegraph_tensor(wo)
    wgb.destroy_wholegraph_tensor(wi)
    wgb.destroy_embedding(emb)
    wgb.destroy_cache_policy(policy)


@pytest.mark.parametrize("mem_name", ["MtContinuous", "MtDistributed"])
def test_device_cache_in_front_of_a_host_table(gpu, wgb, orc, comm, mem_name):
    """The mode a same-communicator cache exists for in the reference (device_cached_host_embedding,
    cpp/src/wholegraph/embedding.cpp:567-759): the table lives in pinned host memory, the cache lines
    in device memory.  Cached gathers return the table's rows across LFU updates, training goes
    through the cache, and the write-back puts the trained rows into the host table."""
    import torch
    MT, ML = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation
    mem = getattr(MT, mem_name)
    rows, dim, ratio = 4096, 48, 0.25
    rng = np.random.default_rng(17)
    emb, policy = _make(gpu, wgb, comm, rows, dim, torch.float32, ratio, mem_type=mem, cache_type=mem,
                        table_location=ML.MlHost)
    table = wgb.embedding_tensor(emb)
    handle = C.c_void_p(wgb.lib().wholegraph_tensor_get_memory_handle(table))
    assert wgb.lib().wholegraph_get_memory_location(handle) == int(ML.MlHost)
    lines_handle = C.c_void_p(wgb.lib().wholegraph_tensor_get_memory_handle(wgb.embedding_cache_tensors(emb)[2]))
    assert wgb.lib().wholegraph_get_memory_location(lines_handle) == int(ML.MlDevice)
    init = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    gpu.scatter(torch.from_numpy(init).cuda(), torch.arange(rows, device="cuda", dtype=torch.int64), table)
    torch.cuda.synchronize()
    for step in range(4):
        ids = _zipf_like(rng, rows, 4000).astype(np.int64)
        out = _forward(gpu, wgb, torch, emb, ids, dim, torch.float32, step != 2)
        assert np.array_equal(out.cpu().numpy(), init[ids]), f"step {step}"
    tags_t = wgb.embedding_cache_tensors(emb)[0]
    sets = wgb.lib().wholegraph_tensor_get_tensor_description(tags_t).contents.sizes[0]
    tags = _read_tensor(gpu, torch, tags_t, sets, 32, torch.int16).cpu().numpy().view(np.uint16)
    assert (tags & VALID).sum() > 32, "nothing was cached"
    # train through the cache, then write back into the host table
    opt = wgb.create_optimizer(wgb.WholeGraphOptimizerType.OptSgd)
    wgb.check(wgb.lib().wholegraph_embedding_set_optimizer(emb, opt), "set_optimizer")
    want = init.copy()
    for step in range(2):
        ids = _zipf_like(rng, rows, 3000).astype(np.int64)
        grads = rng.uniform(-1, 1, size=(len(ids), dim)).astype(np.float32)
        d_ids, d_grads = torch.from_numpy(ids).cuda(), torch.from_numpy(grads).cuda()
        wi, wg = gpu.wrap_torch_tensor(d_ids), gpu.wrap_torch_tensor(d_grads)
        wgb.EmbeddingGatherGradientApply(emb, wi, wg, True, 0.05, wgb.cached_env_fns(), gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wg)
        uniq, sums = orc.dedup_gradients(ids, grads, block=256)
        orc.optimizer_apply(1, uniq, sums, want, lr=0.05)
    all_ids = np.arange(rows, dtype=np.int64)
    assert np.array_equal(_forward(gpu, wgb, torch, emb, all_ids, dim, torch.float32, False).cpu().numpy(), want)
    wgb.embedding_writeback_all_cache(emb)
    assert np.array_equal(_read_tensor(gpu, torch, table, rows, dim, torch.float32).cpu().numpy(), want)
    wgb.destroy_embedding(emb)
    wgb.lib().wholegraph_destroy_embedding_optimizer(opt)
    wgb.destroy_cache_policy(policy)


@pytest.mark.parametrize("mem_name", ["MtContinuous", "MtDistributed"])
@pytest.mark.parametrize("dtype_name,dim", [("f32", 32), ("bf16", 100)])
def test_read_only_cache_on_its_own_communicator(gpu, wgb, orc, comm, mem_name, dtype_name, dim):
    """A cache on another communicator than its table - every group of ranks caching the whole table
    for itself, read-only (reference: local_cached_global_readonly_embedding, cpp/src/wholegraph/
    embedding.cpp:761-884; creation rules :972-987).  The LFU update only decides which rows get which
    lines; the rows come from the table through wholegraph_gather and go into the lines through a
    scatter; a lookup copies hits from the lines and leaves the misses to a second gather.  On one
    GPU both communicators have one rank, but they are different objects, which is what selects
    this path."""
    import torch
    MT, ML, AT, DT = (wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphAccessType,
                      wgb.WholeGraphDataType)
    dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    cache_comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    rows, ratio = 5000, 0.25                       # coverage 128
    rng = np.random.default_rng(dim)
    lib = wgb.lib()
    desc = wgb.make_description([rows, dim], DT(gpu.TORCH_TO_WG[dtype]))
    # what the reference refuses: a cache of this kind that is not CONTINUOUS or not read-only
    for bad_type, bad_access in ((MT.MtDistributed, AT.AtReadOnly), (MT.MtContinuous, AT.AtReadWrite)):
        bad = wgb.create_cache_policy(cache_comm, bad_type, ML.MlDevice, bad_access, ratio)
        e = C.c_void_p()
        rc = lib.wholegraph_create_embedding(C.byref(e), C.byref(desc), comm, int(getattr(MT, mem_name)), int(ML.MlDevice),
                                             bad, None, -1, 0)
        assert rc == int(wgb.ErrorCode.INVALID_INPUT)
        wgb.destroy_cache_policy(bad)
    policy = wgb.create_cache_policy(cache_comm, MT.MtContinuous, ML.MlDevice, AT.AtReadOnly, ratio)
    emb = wgb.create_embedding(desc, comm, getattr(MT, mem_name), ML.MlDevice, cache_policy=policy)
    table = wgb.embedding_tensor(emb)
    tags_t, lfu_t, lines_t, coverage = wgb.embedding_cache_tensors(emb)
    assert coverage == 128
    table_rows = lib.wholegraph_tensor_get_tensor_description(table).contents.sizes[0]
    init = torch.from_numpy(rng.uniform(-1, 1, size=(table_rows, dim)).astype(np.float32)).cuda().to(dtype)
    gpu.scatter(init, torch.arange(table_rows, device="cuda", dtype=torch.int64), table)
    torch.cuda.synchronize()
    sets = lib.wholegraph_tensor_get_tensor_description(tags_t).contents.sizes[0]
    assert sets == -(-table_rows // coverage)
    model = orc.CachePolicyModel(sets * coverage, coverage)
    for step in range(6):
        ids = _zipf_like(rng, rows, 3000).astype(np.int64)
        if step == 4:
            ids[::17] = -1                                       # skipped positions keep what the output held
        adjust = step != 3
        d_ids = torch.from_numpy(ids).cuda()
        out = torch.full((len(ids), dim), 9, dtype=dtype, device="cuda")
        wi, wo = gpu.wrap_torch_tensor(d_ids), gpu.wrap_torch_tensor(out)
        wgb.EmbeddingGatherForward(emb, wi, wo, adjust, wgb.cached_env_fns(), gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wo)
        want = init[torch.from_numpy(np.where(ids < 0, 0, ids)).cuda()]
        want[torch.from_numpy(ids < 0).cuda()] = 9
        assert torch.equal(out, want), f"step {step}"
        if adjust:
            model.update(ids[ids >= 0])
        tags = _read_tensor(gpu, torch, tags_t, sets, 32, torch.int16).cpu().numpy().view(np.uint16)
        for s_ in range(sets):
            got = {int(t & ROW_MASK): line for line, t in enumerate(tags[s_]) if t & VALID}
            assert got == model.cached.get(s_, {}), f"step {step} set {s_}"
        assert not (tags & MODIFIED).any()
        esz = init.element_size()
        pad = -(-dim // (16 // esz)) * (16 // esz)
        lines = _read_tensor(gpu, torch, lines_t, sets * 32, pad, dtype)
        s_idx, l_idx = np.nonzero(tags & VALID)
        src_rows = s_idx * coverage + (tags[s_idx, l_idx] & ROW_MASK)
        assert torch.equal(lines[torch.from_numpy(s_idx * 32 + l_idx).cuda(), :dim],
                           init[torch.from_numpy(src_rows.astype(np.int64)).cuda()]), "a line holds the wrong row"
    assert sum(len(v) for v in model.cached.values()) > 32
    # read-only: it cannot be trained, and dropping the cache leaves gathers correct
    opt = wgb.create_optimizer(wgb.WholeGraphOptimizerType.OptSgd)
    assert lib.wholegraph_embedding_set_optimizer(emb, opt) == int(wgb.ErrorCode.NOT_SUPPORTED)
    lib.wholegraph_destroy_embedding_optimizer(opt)
    wgb.embedding_drop_all_cache(emb)
    assert not _read_tensor(gpu, torch, tags_t, sets, 32, torch.int16).cpu().numpy().any()
    ids = _zipf_like(rng, rows, 500).astype(np.int64)
    out = _forward(gpu, wgb, torch, emb, ids, dim, dtype, False)
    assert torch.equal(out, init[torch.from_numpy(ids).cuda()])
    wgb.destroy_embedding(emb)
    wgb.destroy_cache_policy(policy)
    wgb.destroy_communicator(cache_comm)
