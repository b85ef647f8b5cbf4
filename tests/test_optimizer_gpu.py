"""GPU parity of wholegraph_embedding_gather_gradient_apply (duplicate-gradient sum fused with
SGD / Lazy Adam / AdaGrad / RMSProp) against the CPU oracle, through the C ABI.

Grid after the reference's gradient-apply tests
(cpp/tests/wholegraph_tensor_ops/wholegraph_embedding_gradient_apply_tests.cu:798-1007): four
optimizers, dims 3/4/32/64/127/129/392, int32 and int64 ids, fp32 / fp16 / bf16 tables, several
steps with duplicate ids.  The kernels round every operation separately in the oracle's order,
so weights and states must match bit for bit (the required bound is 1e-6 relative)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

OPTS = {"sgd": 1, "adam": 2, "rmsprop": 3, "adagrad": 4}


@pytest.fixture(scope="module")
def comm(gpu, wgb):
    c = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    yield c
    wgb.destroy_communicator(c)


def _host_bits(torch, t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def _read_all(gpu, torch, wg_tensor, rows, dim, dtype):
    ids = torch.arange(rows, device="cuda", dtype=torch.int64)
    out = torch.empty((rows, dim), dtype=dtype, device="cuda")
    gpu.gather(wg_tensor, ids, out)
    torch.cuda.synchronize()
    return out


def _run(gpu, wgb, orc, comm, opt_name, rows, dim, table_dtype, idx_dtype, steps, n, params, mem_type, block=0,
         cache_ratio=None):
    import torch
    DT, MT, ML = wgb.WholeGraphDataType, wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[table_dtype]
    wg_dt = gpu.TORCH_TO_WG[tdt]
    rng = np.random.default_rng(hash((opt_name, dim, table_dtype)) % (2 ** 31))
    env = wgb.cached_env_fns()
    policy = None
    if cache_ratio is not None:   # train through a set-associative cache in front of table and state
        policy = wgb.create_cache_policy(comm, mem_type, ML.MlDevice, wgb.WholeGraphAccessType.AtReadWrite,
                                         cache_ratio)
    emb = wgb.create_embedding(wgb.make_description([rows, dim], DT(wg_dt)), comm, mem_type, ML.MlDevice,
                               cache_policy=policy)
    opt = wgb.create_optimizer(wgb.WholeGraphOptimizerType(OPTS[opt_name]), **params)
    wgb.check(wgb.lib().wholegraph_embedding_set_optimizer(emb, opt), "set_optimizer")
    table = wgb.embedding_tensor(emb)

    init = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    d_init = torch.from_numpy(init).cuda().to(tdt)
    gpu.scatter(d_init, torch.arange(rows, device="cuda", dtype=torch.int64), table)
    torch.cuda.synchronize()
    # host mirrors
    w_host = np.ascontiguousarray(_host_bits(torch, d_init))
    padded = -(-dim // (16 // d_init.element_size())) * (16 // d_init.element_size())
    n_states = {"sgd": 0, "adam": 2, "rmsprop": 1, "adagrad": 1}[opt_name]
    state_host = np.zeros((rows, max(n_states, 1) * padded), dtype=np.float32)
    beta_host = np.ones((rows, 2), dtype=np.float32)

    lr = 0.01
    for step in range(steps):
        idx = rng.integers(0, rows, size=n)
        idx[: n // 4] = idx[n // 2: n // 2 + n // 4]  # plenty of duplicates
        idx = idx.astype(idx_dtype)
        grads = rng.uniform(-1, 1, size=(n, dim)).astype(np.float32)
        d_idx, d_grads = torch.from_numpy(idx).cuda(), torch.from_numpy(grads).cuda()  # keep them alive
        wi, wg = gpu.wrap_torch_tensor(d_idx), gpu.wrap_torch_tensor(d_grads)
        wgb.EmbeddingGatherGradientApply(emb, wi, wg, policy is not None and step != 2, lr, env,
                                         gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wg)
        uniq, sums = orc.dedup_gradients(idx, grads, block=block)
        orc.optimizer_apply(OPTS[opt_name], uniq, sums, w_host, lr=lr,
                            state=state_host if n_states else None, v_offset=padded,
                            beta12t=beta_host if opt_name == "adam" else None,
                            weights_bf16=(table_dtype == "bf16"),
                            weight_decay=params.get("weight_decay", 0.0), epsilon=params.get("epsilon", 1e-8),
                            beta1=params.get("beta1", 0.9), beta2=params.get("beta2", 0.999),
                            alpha=params.get("alpha", 0.99), adam_w=params.get("adam_w", 0.0) > 0.5)

    if policy is not None:
        # a gather through the cache sees the trained rows before anything is written back ...
        ids = torch.arange(rows, device="cuda", dtype=torch.int64)
        out = torch.empty((rows, dim), dtype=tdt, device="cuda")
        wi, wo = gpu.wrap_torch_tensor(ids), gpu.wrap_torch_tensor(out)
        wgb.EmbeddingGatherForward(emb, wi, wo, False, env, gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wo)
        assert np.array_equal(_host_bits(torch, out).view(w_host.dtype), w_host), "cached gather differs"
        tags = wgb.embedding_cache_tensors(emb)[0]
        sets = wgb.lib().wholegraph_tensor_get_tensor_description(tags).contents.sizes[0]
        bits = _read_all(gpu, torch, tags, sets, 32, torch.int16).cpu().numpy().view(np.uint16)
        assert (bits & 0x8000).any(), "training never touched a cache line"
        # ... and the tables hold them after the write-back
        wgb.embedding_writeback_all_cache(emb)
        bits = _read_all(gpu, torch, tags, sets, 32, torch.int16).cpu().numpy().view(np.uint16)
        assert not (bits & 0x8000).any()
    got_w = _host_bits(torch, _read_all(gpu, torch, table, rows, dim, tdt))
    assert np.array_equal(got_w.view(w_host.dtype), w_host), "weights differ from the oracle"
    names = wgb.embedding_state_names(emb)
    assert names == {"sgd": [], "adam": ["m", "v", "beta12t"], "rmsprop": ["v"], "adagrad": ["state_sum"]}[opt_name]
    for k, name in enumerate([x for x in names if x != "beta12t"]):
        st = _read_all(gpu, torch, wgb.embedding_state(emb, name), rows, dim, torch.float32).cpu().numpy()
        assert np.array_equal(st, state_host[:, k * padded:k * padded + dim]), f"state {name} differs"
    if opt_name == "adam":
        b = _read_all(gpu, torch, wgb.embedding_state(emb, "beta12t"), rows, 2, torch.float32).cpu().numpy()
        assert np.array_equal(b, beta_host)
    wgb.destroy_embedding(emb)
    wgb.lib().wholegraph_destroy_embedding_optimizer(opt)
    if policy is not None:
        wgb.destroy_cache_policy(policy)


@pytest.mark.parametrize("opt_name,params", [("sgd", {}), ("sgd", {"weight_decay": 0.1}),
                                             ("adam", {}), ("adam", {"weight_decay": 0.05, "adam_w": 1.0}),
                                             ("adam", {"weight_decay": 0.05, "beta1": 0.8, "epsilon": 1e-6}),
                                             ("adagrad", {"weight_decay": 0.01}), ("rmsprop", {"alpha": 0.9})])
@pytest.mark.parametrize("dim", [3, 4, 32, 64, 127, 129, 392])
def test_gradient_apply_fp32(gpu, wgb, orc, comm, opt_name, params, dim):
    _run(gpu, wgb, orc, comm, opt_name, 4096, dim, "f32", np.int64, 3, 3000, params,
         wgb.WholeGraphMemoryType.MtDistributed)


@pytest.mark.parametrize("opt_name", ["sgd", "adam", "adagrad", "rmsprop"])
@pytest.mark.parametrize("table_dtype", ["f16", "bf16"])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_gradient_apply_half_tables(gpu, wgb, orc, comm, opt_name, table_dtype, idx_dtype):
    _run(gpu, wgb, orc, comm, opt_name, 2048, 100, table_dtype, idx_dtype, 3, 1500, {},
         wgb.WholeGraphMemoryType.MtContinuous)


def test_gradient_apply_ten_steps_long_chains(gpu, wgb, orc, comm):
    """Ten Lazy Adam steps on a small table so that every row is hit many times per step
    (duplicate chains of ~40 rows), dim 256 as in the sparse-Adam configuration."""
    _run(gpu, wgb, orc, comm, "adam", 256, 256, "f32", np.int64, 10, 10_000, {},
         wgb.WholeGraphMemoryType.MtDistributed)


@pytest.mark.parametrize("opt_name", ["adam", "sgd"])
@pytest.mark.parametrize("dim", [256, 30])
def test_gradient_apply_runs_longer_than_a_block(gpu, wgb, orc, comm, opt_name, dim):
    """Ids that occur more than WHOLEGRAPH_B200_DEDUP_BLOCK (256) times in one call: the kernels sum
    such a run block by block; the oracle restates exactly that order (block=256), so the result
    is still bit-exact.  12 rows, 20,000 gradient rows per step: every run is ~1,700 long."""
    _run(gpu, wgb, orc, comm, opt_name, 12, dim, "f32", np.int64, 3, 20_000, {},
         wgb.WholeGraphMemoryType.MtDistributed, block=256)


def test_blocked_sum_stays_close_to_the_single_chain(gpu, orc):
    """How far the block-by-block order moves a long run's sum from the reference's single chain:
    bounded by fp32 summation error, far below the gradients' own scale."""
    rng = np.random.default_rng(0)
    n, dim = 200_000, 16
    idx = np.zeros(n, dtype=np.int64)
    grads = rng.normal(0, 1e-3, size=(n, dim)).astype(np.float32)
    _, chain = orc.dedup_gradients(idx, grads)
    _, blocked = orc.dedup_gradients(idx, grads, block=256)
    exact = grads.astype(np.float64).sum(axis=0)
    scale = np.abs(grads).sum(axis=0)            # the natural error scale of a sum
    assert np.all(np.abs(chain[0] - blocked[0]) <= 1e-6 * scale)
    assert np.all(np.abs(blocked[0] - exact) <= np.abs(chain[0] - exact) + 1e-7 * scale)


def test_optimizer_parameter_names(gpu, wgb):
    import ctypes as C
    o = wgb.create_optimizer(wgb.WholeGraphOptimizerType.OptSgd)
    v = C.c_float(0.5)
    assert wgb.lib().wholegraph_optimizer_set_parameter(o, b"weight_decay", C.byref(v)) == 0
    assert wgb.lib().wholegraph_optimizer_set_parameter(o, b"beta1", C.byref(v)) == int(wgb.ErrorCode.INVALID_INPUT)
    wgb.lib().wholegraph_destroy_embedding_optimizer(o)


@pytest.mark.parametrize("rr,rows", [(4, 1003), (16, 4096), (7, 50)])
def test_round_robin_embedding_gather_and_apply(gpu, wgb, orc, comm, rr, rows):
    """An embedding created with round_robin_size != 0: ids are remapped before every gather and
    gradient apply (reference: cpp/src/wholegraph_tensor_ops/functions/map_indices_func.cu:16-34,
    reached from cpp/src/wholegraph/embedding.cpp:1027-1087) and the table is sized so that every rank
    stores the same number of rows (embedding.cpp:459-476).  Gather returns the rows the oracle's
    literal restatement of the remap names; one SGD step lands on those rows and no others."""
    import torch
    DT, MT, ML = wgb.WholeGraphDataType, wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation
    dim, world = 24, 1
    env = wgb.cached_env_fns()
    emb = wgb.create_embedding(wgb.make_description([rows, dim], DT.DtFloat), comm, MT.MtContinuous, ML.MlDevice,
                               round_robin_size=rr)
    table = wgb.embedding_tensor(emb)
    extra = min(rows % (world * rr), rr)
    stored = (rows // (world * rr) * rr + extra) * world
    got_rows = wgb.lib().wholegraph_tensor_get_tensor_description(table).contents.sizes[0]
    assert got_rows == stored
    rng = np.random.default_rng(rr)
    init = rng.uniform(-1, 1, size=(stored, dim)).astype(np.float32)
    gpu.scatter(torch.from_numpy(init).cuda(), torch.arange(stored, device="cuda", dtype=torch.int64), table)
    for idx_dtype in (np.int64, np.int32):
        ids = rng.integers(0, stored, size=777).astype(idx_dtype)
        mapped = orc.round_robin_map(ids, rr=rr, world=world, entry_start=0)
        d_ids = torch.from_numpy(ids).cuda()
        out = torch.zeros((len(ids), dim), dtype=torch.float32, device="cuda")
        wi, wo = gpu.wrap_torch_tensor(d_ids), gpu.wrap_torch_tensor(out)
        wgb.EmbeddingGatherForward(emb, wi, wo, False, env, gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wo)
        assert np.array_equal(out.cpu().numpy(), init[mapped])
    # one SGD step through the remap
    opt = wgb.create_optimizer(wgb.WholeGraphOptimizerType.OptSgd)
    wgb.check(wgb.lib().wholegraph_embedding_set_optimizer(emb, opt), "set_optimizer")
    ids = rng.integers(0, stored, size=500).astype(np.int64)
    grads = rng.uniform(-1, 1, size=(len(ids), dim)).astype(np.float32)
    d_ids, d_grads = torch.from_numpy(ids).cuda(), torch.from_numpy(grads).cuda()
    wi, wg = gpu.wrap_torch_tensor(d_ids), gpu.wrap_torch_tensor(d_grads)
    wgb.EmbeddingGatherGradientApply(emb, wi, wg, False, 0.1, env, gpu.current_stream_int())
    torch.cuda.synchronize()
    wgb.destroy_wholegraph_tensor(wi)
    wgb.destroy_wholegraph_tensor(wg)
    want = init.copy()
    uniq, sums = orc.dedup_gradients(orc.round_robin_map(ids, rr=rr, world=world, entry_start=0), grads)
    orc.optimizer_apply(1, uniq, sums, want, lr=0.1)
    got = _read_all(gpu, torch, table, stored, dim, torch.float32).cpu().numpy()
    assert np.array_equal(got, want)
    wgb.destroy_embedding(emb)
    wgb.lib().wholegraph_destroy_embedding_optimizer(opt)


@pytest.mark.parametrize("switches", [{}, {"WG_SYNC_FREE": "0"}, {"WG_SYNC_FREE": "0", "WG_PEER_GRADIENT": "1"},
                                      {"WG_GRADIENT_PRESUM": "0"}],
                         ids=["merged", "presum-exchange", "presum-peer-push", "every-row-routed"])
@pytest.mark.parametrize("opt_name,table_dtype,dim", [("adam", "f32", 256), ("adam", "f32", 33), ("sgd", "bf16", 100),
                                                      ("adagrad", "f16", 64), ("rmsprop", "f32", 392)])
def test_multi_rank_gradient_code_on_one_rank(gpu, wgb, orc, monkeypatch, switches, opt_name, table_dtype, dim):
    """WG_SINGLE_RANK_EXCHANGE=1: a one-rank communicator runs the multi-rank gradient path - the
    per-rank pre-sum left in the exchange arena and the owner's merge (bitmaps, ranks, one warp per
    touched row reading the senders' sums), or the routed variants the other switches select - with
    itself as its only peer, so that this code is checked against the oracle on one GPU as well."""
    monkeypatch.setenv("WG_SINGLE_RANK_EXCHANGE", "1")
    for k, v in switches.items():
        monkeypatch.setenv(k, v)
    c = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    try:
        _run(gpu, wgb, orc, c, opt_name, 4096, dim, table_dtype, np.int64, 3, 3000, {"weight_decay": 0.01},
             wgb.WholeGraphMemoryType.MtDistributed, block=256)
    finally:
        wgb.destroy_communicator(c)


def test_merged_gradient_path_with_a_run_longer_than_a_block(gpu, wgb, orc, monkeypatch):
    """One id takes a third of 6,000 gradient rows: the sender's pre-sum cuts it into blocks of 256,
    the owner's merge then sees one row of sums for it."""
    import torch
    monkeypatch.setenv("WG_SINGLE_RANK_EXCHANGE", "1")
    c = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    DT, MT, ML = wgb.WholeGraphDataType, wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation
    rows, dim, n = 3000, 64, 6000
    rng = np.random.default_rng(4)
    env = wgb.cached_env_fns()
    emb = wgb.create_embedding(wgb.make_description([rows, dim], DT.DtFloat), c, MT.MtDistributed, ML.MlDevice)
    opt = wgb.create_optimizer(wgb.WholeGraphOptimizerType.OptLazyAdam)
    wgb.check(wgb.lib().wholegraph_embedding_set_optimizer(emb, opt), "set_optimizer")
    table = wgb.embedding_tensor(emb)
    init = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    gpu.scatter(torch.from_numpy(init).cuda(), torch.arange(rows, device="cuda", dtype=torch.int64), table)
    w, state, beta = init.copy(), np.zeros((rows, 2 * dim), np.float32), np.ones((rows, 2), np.float32)
    for step in range(2):
        ids = rng.integers(0, rows, size=n).astype(np.int64)
        ids[rng.permutation(n)[: n // 3]] = 1234
        grads = rng.uniform(-1, 1, size=(n, dim)).astype(np.float32)
        d_ids, d_grads = torch.from_numpy(ids).cuda(), torch.from_numpy(grads).cuda()
        wi, wg = gpu.wrap_torch_tensor(d_ids), gpu.wrap_torch_tensor(d_grads)
        wgb.EmbeddingGatherGradientApply(emb, wi, wg, False, 0.01, env, gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wg)
        uniq, sums = orc.dedup_gradients(ids, grads, block=256)
        orc.optimizer_apply(2, uniq, sums, w, lr=0.01, state=state, v_offset=dim, beta12t=beta)
    assert np.array_equal(_read_all(gpu, torch, table, rows, dim, torch.float32).cpu().numpy(), w)
    assert np.array_equal(_read_all(gpu, torch, wgb.embedding_state(emb, "m"), rows, dim, torch.float32).cpu().numpy(), state[:, :dim])
    assert np.array_equal(_read_all(gpu, torch, wgb.embedding_state(emb, "v"), rows, dim, torch.float32).cpu().numpy(), state[:, dim:])
    assert np.array_equal(_read_all(gpu, torch, wgb.embedding_state(emb, "beta12t"), rows, 2, torch.float32).cpu().numpy(), beta)
    wgb.destroy_embedding(emb)
    wgb.lib().wholegraph_destroy_embedding_optimizer(opt)
    wgb.destroy_communicator(c)
