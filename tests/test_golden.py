"""Committed golden vectors (tests/golden/golden_small.npz, made by tests/golden/make_golden.py):
the CPU oracle must still produce them (no GPU), and the CUDA path must reproduce them bit for
bit through the C ABI (GPU)."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_small.npz")


@pytest.fixture(scope="module")
def g():
    return dict(np.load(GOLDEN))


def test_oracle_reproduces_golden(orc, g):
    t, idx = g["gather_table_f32"], g["gather_idx"]
    assert np.array_equal(orc.gather(t, idx, out_dt=2), g["gather_out_f16"])
    assert np.array_equal(orc.gather(t, idx, out_dt=4), g["gather_out_bf16"])
    assert np.array_equal(orc.gather(t, idx, out_dt=3), g["gather_out_f64"])
    assert np.array_equal(orc.scatter(g["scatter_rows_f16"], g["scatter_idx"], t.copy()), g["scatter_table_after"])
    assert np.array_equal(orc.gather(g["int_table"], g["int_idx"], out_dt=8), g["int_out_i8"])
    w = g["adam_w0"].copy()
    rows, dim = w.shape
    state, beta = np.zeros((rows, 2 * dim), np.float32), np.ones((rows, 2), np.float32)
    for step in range(3):
        uniq, sums = orc.dedup_gradients(g[f"adam_ids_{step}"], g[f"adam_grads_{step}"])
        orc.optimizer_apply(orc.OPT_LAZY_ADAM, uniq, sums, w, lr=1e-3, state=state, v_offset=dim, beta12t=beta)
    assert np.array_equal(w, g["adam_w3"]) and np.array_equal(state, g["adam_state3"])
    assert np.array_equal(beta, g["adam_beta3"])


@pytest.mark.gpu
def test_cuda_path_reproduces_golden(gpu, wgb, g):
    import torch
    t = torch.from_numpy(g["gather_table_f32"]).cuda()
    idx = torch.from_numpy(g["gather_idx"]).cuda()
    wt = gpu.wrap_torch_tensor(t)
    n, dim = idx.numel(), t.shape[1]
    for key, dt in (("gather_out_f16", torch.float16), ("gather_out_bf16", torch.bfloat16), ("gather_out_f64", torch.float64)):
        out = torch.zeros((n, dim), dtype=dt, device="cuda")
        gpu.gather(wt, idx, out)
        torch.cuda.synchronize()
        got = out.view(torch.int16).cpu().numpy().view(np.uint16) if dt == torch.bfloat16 else out.cpu().numpy()
        assert np.array_equal(got, g[key]), key
    gpu.scatter(torch.from_numpy(g["scatter_rows_f16"]).cuda(), torch.from_numpy(g["scatter_idx"]).cuda(), wt)
    torch.cuda.synchronize()
    assert np.array_equal(t.cpu().numpy(), g["scatter_table_after"])
    wgb.destroy_wholegraph_tensor(wt)
    it, iidx = torch.from_numpy(g["int_table"]).cuda(), torch.from_numpy(g["int_idx"]).cuda()
    wi = gpu.wrap_torch_tensor(it)
    for key, dt in (("int_out_i8", torch.int8), ("int_out_i32", torch.int32)):
        out = torch.zeros((iidx.numel(), it.shape[1]), dtype=dt, device="cuda")
        gpu.gather(wi, iidx, out)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), g[key]), key
    wgb.destroy_wholegraph_tensor(wi)
    # three Lazy Adam steps through the embedding API
    comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    rows, dim = g["adam_w0"].shape
    emb = wgb.create_embedding(wgb.make_description([rows, dim], wgb.WholeGraphDataType.DtFloat), comm,
                               wgb.WholeGraphMemoryType.MtDistributed, wgb.WholeGraphMemoryLocation.MlDevice)
    opt = wgb.create_optimizer(wgb.WholeGraphOptimizerType.OptLazyAdam)
    wgb.check(wgb.lib().wholegraph_embedding_set_optimizer(emb, opt), "set_optimizer")
    table = wgb.embedding_tensor(emb)
    all_ids = torch.arange(rows, device="cuda", dtype=torch.int64)
    gpu.scatter(torch.from_numpy(g["adam_w0"]).cuda(), all_ids, table)
    for step in range(3):
        d_ids, d_grads = torch.from_numpy(g[f"adam_ids_{step}"]).cuda(), torch.from_numpy(g[f"adam_grads_{step}"]).cuda()
        wi, wg = gpu.wrap_torch_tensor(d_ids), gpu.wrap_torch_tensor(d_grads)
        wgb.EmbeddingGatherGradientApply(emb, wi, wg, False, 1e-3, wgb.cached_env_fns(), gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wg)
    w = torch.empty((rows, dim), dtype=torch.float32, device="cuda")
    gpu.gather(table, all_ids, w)
    m = torch.empty((rows, dim), dtype=torch.float32, device="cuda")
    gpu.gather(wgb.embedding_state(emb, "m"), all_ids, m)
    torch.cuda.synchronize()
    assert np.array_equal(w.cpu().numpy(), g["adam_w3"])
    assert np.array_equal(m.cpu().numpy(), g["adam_state3"][:, :dim])
    wgb.destroy_embedding(emb)
    wgb.lib().wholegraph_destroy_embedding_optimizer(opt)
    wgb.destroy_communicator(comm)
