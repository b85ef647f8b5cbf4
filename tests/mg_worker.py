"""One rank of the multi-GPU parity tests (started by tests/test_multi_gpu.py, one process per GPU).

Rendezvous is a file: rank 0 writes the communicator's unique id, the others read it.  Every
scenario compares against the CPU oracle evaluated on a closed-form table that each rank can
rebuild on the host.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def table_values(rows, dim, np_dtype):
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(dim, dtype=np.int64)[None, :]
    if np.issubdtype(np_dtype, np.integer):
        return ((r * 131 + c * 7) % 20011 - 10000).astype(np_dtype)
    return (((r * 131 + c * 7) % 2001 - 1000) / 1000.0).astype(np.float32).astype(np_dtype)


def main():
    rank, world, rdv = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    scenarios = sys.argv[4].split(",")
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("WG_TEST_STACK_AFTER", "90")) * len(scenarios), exit=True)
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    wgb = pkg.binding
    from cugraph_gnn_b200 import torch_utils as tu
    from oracle import oracle as orc
    wgb.load_library()
    torch.cuda.set_device(rank)
    wgb.init(0, int(os.environ.get("WG_TEST_LOG_LEVEL", "2")))

    uid_path = os.path.join(rdv, "uid.bin")
    if rank == 0:
        raw = wgb.unique_id_to_bytes(wgb.create_unique_id())
        with open(uid_path + ".tmp", "wb") as f:
            f.write(raw)
        os.rename(uid_path + ".tmp", uid_path)
    else:
        deadline = time.time() + 120
        while not os.path.exists(uid_path):
            if time.time() > deadline:
                raise RuntimeError("rendezvous file never appeared")
            time.sleep(0.05)
        with open(uid_path, "rb") as f:
            raw = f.read()
    comm = wgb.create_communicator(wgb.unique_id_from_bytes(raw), rank, world)
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    env = wgb.cached_env_fns()

    def make_table(mem_type, rows, dim, tdt, partition=None, location=ML.MlDevice):
        desc = wgb.make_description([rows, dim], DT(tu.TORCH_TO_WG[tdt]))
        t = wgb.create_wholegraph_tensor(desc, comm, mem_type, location, partition)
        start, count = wgb.C.c_size_t(), wgb.C.c_size_t()
        wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_start(wgb.C.byref(start), t), "entry_start")
        wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_count(wgb.C.byref(count), t), "entry_count")
        npdt = np.float32 if tdt in (torch.float32, torch.float16, torch.bfloat16) else np.int64
        full = table_values(rows, dim, npdt)
        local = torch.from_numpy(full[start.value:start.value + count.value]).cuda().to(tdt).contiguous()
        tu.write_local_shard(t, local)
        torch.cuda.synchronize()
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        return t, full

    def host_table(full, tdt):
        if tdt == torch.float16:
            return full.astype(np.float16), False
        if tdt == torch.bfloat16:
            return orc.float_to_bf16_bits(full), True
        return full, False

    def to_host(t):
        return t.view(torch.int16).cpu().numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.cpu().numpy()

    def check_gather(mem_type, rows, dim, tdt, odt, n, partition=None, idx_dtype=torch.int64, seed=0,
                     location=ML.MlDevice):
        if isinstance(n, (list, tuple)):       # a different request length on every rank
            n = n[rank % len(n)]
        print(f"rank {rank}: gather {mem_type.name} rows={rows} dim={dim} {tdt}->{odt} n={n}", flush=True)
        t, full = make_table(mem_type, rows, dim, tdt, partition, location)
        g = torch.Generator(device="cuda").manual_seed(1000 * seed + rank)
        idx = torch.randint(0, rows, (n,), generator=g, device="cuda").to(idx_dtype)
        if n > 10:
            idx[::37] = -1
        out = torch.full((n, dim), 3, dtype=odt, device="cuda")
        tu.gather(t, idx, out, env)
        torch.cuda.synchronize()
        tab, tab_bf16 = host_table(full, tdt)
        want = np.full((n, dim), 3, dtype=np.float32)
        want = to_host(torch.from_numpy(want).to(odt)) if odt != torch.float32 else want
        want = np.ascontiguousarray(want)
        orc.gather(tab, idx.cpu().numpy(), out_dt=int(tu.TORCH_TO_WG[odt]), out=want, table_bf16=tab_bf16)
        got = to_host(out)
        assert np.array_equal(got.view(want.dtype), want), f"gather {mem_type.name} {tdt}->{odt} n={n} differs on rank {rank}"
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        wgb.destroy_wholegraph_tensor(t)

    def check_scatter(mem_type, rows, dim, tdt, idt, n_per_rank, location=ML.MlDevice):
        print(f"rank {rank}: scatter {mem_type.name} rows={rows} dim={dim} {idt}->{tdt}", flush=True)
        t, full = make_table(mem_type, rows, dim, tdt, None, location)
        # globally unique ids: rank r takes ids congruent to r modulo world
        rng = np.random.default_rng(7)
        perm = rng.permutation(rows)
        n_of = (lambda r: n_per_rank[r % len(n_per_rank)]) if isinstance(n_per_rank, (list, tuple)) else (lambda r: n_per_rank)
        mine = np.ascontiguousarray(perm[rank::world][:n_of(rank)]).astype(np.int64)
        vals = np.random.default_rng(100 + rank).uniform(-1, 1, size=(mine.shape[0], dim)).astype(np.float32)
        d_vals = torch.from_numpy(vals).cuda().to(idt)
        tu.scatter(d_vals, torch.from_numpy(mine).cuda(), t, env)
        torch.cuda.synchronize()
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        # expected table after every rank's scatter
        tab, tab_bf16 = host_table(full, tdt)
        tab = tab.copy()
        for r in range(world):
            ids_r = np.ascontiguousarray(perm[r::world][:n_of(r)]).astype(np.int64)
            vals_r = np.random.default_rng(100 + r).uniform(-1, 1, size=(ids_r.shape[0], dim)).astype(np.float32)
            rows_r = to_host(torch.from_numpy(vals_r).to(idt))
            orc.scatter(np.ascontiguousarray(rows_r), ids_r, tab, rows_bf16=(idt == torch.bfloat16), table_bf16=tab_bf16)
        # read everything back through a gather of all rows
        all_ids = torch.arange(rows, device="cuda", dtype=torch.int64)
        back = torch.empty((rows, dim), dtype=tdt, device="cuda")
        tu.gather(t, all_ids, back, env)
        torch.cuda.synchronize()
        assert np.array_equal(to_host(back).view(tab.dtype), tab), f"scatter {mem_type.name} differs on rank {rank}"
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        wgb.destroy_wholegraph_tensor(t)

    def check_gradient_apply(mem_type, opt_type, opt_code, rows, dim, n, steps, table_dtype=torch.float32,
                             cache_type=None, hot=0, location=ML.MlDevice):
        print(f"rank {rank}: gradient apply {mem_type.name} opt={opt_code} rows={rows} dim={dim} "
              f"cache={cache_type}", flush=True)
        policy = None
        if cache_type is not None:   # rows must already be a multiple of world * 128
            policy = wgb.create_cache_policy(comm, cache_type, ML.MlDevice, wgb.WholeGraphAccessType.AtReadWrite,
                                             0.25)
        emb = wgb.create_embedding(wgb.make_description([rows, dim], DT(tu.TORCH_TO_WG[table_dtype])), comm,
                                   mem_type, location, cache_policy=policy)
        opt = wgb.create_optimizer(opt_type, weight_decay=0.01)
        wgb.check(wgb.lib().wholegraph_embedding_set_optimizer(emb, opt), "set_optimizer")
        table = wgb.embedding_tensor(emb)
        off = orc.equal_partition_offsets(rows, world)
        lo, hi = int(off[rank]), int(off[rank + 1])
        w0 = np.random.default_rng(5).uniform(-1, 1, size=(rows, dim)).astype(np.float32)
        mine = torch.arange(lo, hi, device="cuda", dtype=torch.int64)
        tu.scatter(torch.from_numpy(w0[lo:hi]).cuda().to(table_dtype), mine, table, env)
        torch.cuda.synchronize()
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        w_host = np.ascontiguousarray(to_host(torch.from_numpy(w0).to(table_dtype)))
        es = torch.empty((), dtype=table_dtype).element_size()
        padded = -(-dim // (16 // es)) * (16 // es)
        state = np.zeros((rows, 2 * padded), np.float32)
        beta = np.ones((rows, 2), np.float32)
        for step in range(steps):
            all_ids, all_grads = [], []
            for r in range(world):
                rng = np.random.default_rng(1000 * step + r)
                ids_r = rng.integers(0, rows, size=n).astype(np.int64)
                ids_r[: n // 3] = ids_r[n // 3: 2 * (n // 3)]
                if hot:                       # one id with more duplicates per rank than a summation block
                    ids_r[rng.permutation(n)[:hot]] = rows // 2
                all_ids.append(ids_r)
                all_grads.append(rng.uniform(-1, 1, size=(n, dim)).astype(np.float32))
            d_ids, d_grads = torch.from_numpy(all_ids[rank]).cuda(), torch.from_numpy(all_grads[rank]).cuda()
            wi, wg = tu.wrap_torch_tensor(d_ids), tu.wrap_torch_tensor(d_grads)
            wgb.EmbeddingGatherGradientApply(emb, wi, wg, policy is not None, 0.01, env, tu.current_stream_int())
            torch.cuda.synchronize()
            wgb.destroy_wholegraph_tensor(wi)
            wgb.destroy_wholegraph_tensor(wg)
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            # oracle: every row updated once with the sum of its gradients - by default per-rank sums
            # (arrival order) added in rank order, with WG_GRADIENT_PRESUM=0 one chain in
            # rank-then-arrival order as in the reference (runs over 256 rows block by block)
            if os.environ.get("WG_GRADIENT_PRESUM", "1") == "0":
                uniq, sums = orc.dedup_gradients(np.concatenate(all_ids), np.concatenate(all_grads), block=256)
            else:
                uniq, sums = orc.dedup_gradients_by_rank(all_ids, all_grads)
            orc.optimizer_apply(opt_code, uniq, sums, w_host, lr=0.01, state=state, v_offset=padded, beta12t=beta,
                                weight_decay=0.01, weights_bf16=(table_dtype == torch.bfloat16))
        if policy is not None:
            # forward gathers through the cache see the trained rows (with and without an LFU
            # update), then the write-back puts them into the tables
            for step, adjust in enumerate((True, False, True)):
                ids = np.random.default_rng(77 * step + rank).integers(0, rows // 4, size=4_000).astype(np.int64)
                d_ids = torch.from_numpy(ids).cuda()
                out = torch.empty((len(ids), dim), dtype=table_dtype, device="cuda")
                wi, wo = tu.wrap_torch_tensor(d_ids), tu.wrap_torch_tensor(out)
                wgb.EmbeddingGatherForward(emb, wi, wo, adjust, env, tu.current_stream_int())
                torch.cuda.synchronize()
                wgb.destroy_wholegraph_tensor(wi)
                wgb.destroy_wholegraph_tensor(wo)
                assert np.array_equal(to_host(out).view(w_host.dtype), w_host[ids]), \
                    f"cached gather {step} differs on rank {rank}"
                wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            wgb.embedding_writeback_all_cache(emb)
        got = torch.empty((hi - lo, dim), dtype=table_dtype, device="cuda")
        tu.gather(table, mine, got, env)
        torch.cuda.synchronize()
        assert np.array_equal(to_host(got).view(w_host.dtype), w_host[lo:hi]), f"weights differ on rank {rank}"
        for k, name in enumerate([x for x in wgb.embedding_state_names(emb) if x != "beta12t"]):
            st = torch.empty((hi - lo, dim), dtype=torch.float32, device="cuda")
            tu.gather(wgb.embedding_state(emb, name), mine, st, env)
            torch.cuda.synchronize()
            assert np.array_equal(st.cpu().numpy(), state[lo:hi, k * padded:k * padded + dim]), f"state {name} differs"
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        wgb.destroy_embedding(emb)
        wgb.lib().wholegraph_destroy_embedding_optimizer(opt)
        if policy is not None:
            wgb.destroy_cache_policy(policy)

    def run_fileio():
        # Plain layout: record r of the files is table row r.  Round robin: blocks of rr records are
        # dealt to the ranks in turn (reference: file_io.cpp:100-200).  Every rank stores its shard.
        rows, dim, rr = 1000 * world + 37, 12, 5
        data = np.random.default_rng(9).integers(-2**31, 2**31 - 1, size=(rows, dim), dtype=np.int64).astype(np.int32)
        files = [os.path.join(rdv, f"part_{k}.bin") for k in range(3)]
        cuts = [0, rows // 3 + 1, rows // 3 + 2, rows]
        if rank == 0:
            for k in range(3):
                data[cuts[k]:cuts[k + 1]].tofile(files[k])
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        for mem in (MT.MtContinuous, MT.MtDistributed, MT.MtChunked):
            t, _ = make_table(mem, rows, dim, torch.int32)
            wgb.tensor_from_filelist(t, files)
            ids = torch.arange(rows, device="cuda", dtype=torch.int64)
            got = torch.empty((rows, dim), dtype=torch.int32, device="cuda")
            tu.gather(t, ids, got, env)
            torch.cuda.synchronize()
            assert np.array_equal(got.cpu().numpy(), data), f"plain load {mem.name} differs on rank {rank}"
            out = os.path.join(rdv, f"stored_{mem.name}_{rank}.bin")
            wgb.tensor_to_file(t, out)
            off = orc.equal_partition_offsets(rows, world)
            assert np.array_equal(np.fromfile(out, dtype=np.int32).reshape(-1, dim), data[off[rank]:off[rank + 1]])
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            wgb.destroy_wholegraph_tensor(t)
        # round robin: every rank needs room for its share of the blocks
        per_rank = rows // (world * rr) * rr + rr
        t, _ = make_table(MT.MtDistributed, per_rank * world, dim, torch.int32)
        wgb.tensor_from_filelist(t, files, rr)
        extra = rows % (world * rr)
        mine_n = rows // (world * rr) * rr + max(0, min(rr, extra - rank * rr))
        j = np.arange(mine_n)
        want = data[(j // rr * world + rank) * rr + j % rr]
        local = tu.local_shard_as_torch(t)
        torch.cuda.synchronize()
        assert np.array_equal(local[:mine_n].cpu().numpy(), want), f"round-robin load differs on rank {rank}"
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        wgb.destroy_wholegraph_tensor(t)

    def run_cache():
        OT = wgb.WholeGraphOptimizerType
        rows = 128 * 8 * 5
        check_gradient_apply(MT.MtContinuous, OT.OptLazyAdam, 2, rows, 64, 4_000, 3, cache_type=MT.MtContinuous)
        check_gradient_apply(MT.MtDistributed, OT.OptSgd, 1, rows, 33, 3_000, 3, cache_type=MT.MtDistributed)
        check_gradient_apply(MT.MtChunked, OT.OptAdaGrad, 4, 2 * rows, 100, 3_000, 2, torch.bfloat16,
                             cache_type=MT.MtChunked)

    def run_optimizer():
        OT = wgb.WholeGraphOptimizerType
        check_gradient_apply(MT.MtDistributed, OT.OptLazyAdam, 2, 20_011, 64, 6_000, 3)
        check_gradient_apply(MT.MtContinuous, OT.OptSgd, 1, 5_000, 33, 3_000, 2)
        check_gradient_apply(MT.MtDistributed, OT.OptLazyAdam, 2, 9_000, 32, 4_000, 2, hot=700)
        check_gradient_apply(MT.MtDistributed, OT.OptAdaGrad, 4, 8_000, 100, 3_000, 2, torch.float16)
        check_gradient_apply(MT.MtDistributed, OT.OptRmsProp, 3, 3_000, 256, 9_000, 2, torch.bfloat16)

    def run_memory_type(mem):
        check_gather(mem, 100_003, 128, torch.float16, torch.float16, 50_000, seed=1)
        check_gather(mem, 100_003, 128, torch.float32, torch.float16, 20_001, seed=2)
        check_gather(mem, 40_000, 33, torch.float32, torch.bfloat16, 7_777, idx_dtype=torch.int32, seed=3)
        check_gather(mem, 1_000, 8, torch.int64, torch.int64, 0, seed=4)
        check_gather(mem, 5 * world + 3, 16, torch.bfloat16, torch.float32, 999, seed=5)
        part = [1000 + 10 * r for r in range(world)]
        check_gather(mem, sum(part), 64, torch.float32, torch.float32, 12_345, partition=part, seed=6)
        check_scatter(mem, 30_011, 128, torch.float32, torch.float16, 4_000)
        check_scatter(mem, 9_000, 20, torch.bfloat16, torch.float32, 2_000)

    def run_hosttable():
        # Tables in host memory shared by the ranks: CONTINUOUS / HOST is one POSIX shared-memory
        # segment registered with CUDA on every rank, DISTRIBUTED / HOST pinned memory per rank
        # (reference: memory_handle.cpp:503-546); then the reference's primary cached mode, a device
        # cache in front of a host table (embedding.cpp:567-759), trained through and written back.
        for mem in (MT.MtContinuous, MT.MtDistributed):
            check_gather(mem, 60_007, 128, torch.float32, torch.float16, 9_000, seed=11, location=ML.MlHost)
            check_gather(mem, 10_000, 20, torch.int64, torch.int64, 3_333, idx_dtype=torch.int32, seed=12,
                         location=ML.MlHost)
            check_scatter(mem, 20_011, 64, torch.float32, torch.float16, 3_000, location=ML.MlHost)
        OT = wgb.WholeGraphOptimizerType
        rows = 128 * world * 6
        check_gradient_apply(MT.MtContinuous, OT.OptLazyAdam, 2, rows, 64, 4_000, 3, cache_type=MT.MtContinuous,
                             location=ML.MlHost)
        check_gradient_apply(MT.MtDistributed, OT.OptSgd, 1, rows, 40, 3_000, 2, cache_type=MT.MtDistributed,
                             location=ML.MlHost)

    def run_nodecache():
        # A read-only cache on a smaller communicator than its table: the world is split into two
        # halves (one "node" each) and every half caches the whole DISTRIBUTED table for itself
        # (reference: local_cached_global_readonly_embedding, embedding.cpp:761-884).
        AT = wgb.WholeGraphAccessType
        half = wgb.C.c_void_p()
        color = 0 if rank < (world + 1) // 2 else 1
        wgb.check(wgb.lib().wholegraph_split_communicator(wgb.C.byref(half), comm, color, rank), "split")
        for mem, tdt, dim in ((MT.MtDistributed, torch.float32, 48), (MT.MtContinuous, torch.float16, 128)):
            rows = 128 * world * 7 + 5
            policy = wgb.create_cache_policy(half, MT.MtContinuous, ML.MlDevice, AT.AtReadOnly, 0.25)
            emb = wgb.create_embedding(wgb.make_description([rows, dim], DT(tu.TORCH_TO_WG[tdt])), comm, mem, ML.MlDevice,
                                       cache_policy=policy)
            table = wgb.embedding_tensor(emb)
            trows = wgb.lib().wholegraph_tensor_get_tensor_description(table).contents.sizes[0]
            full = table_values(trows, dim, np.float32)
            start, count = wgb.C.c_size_t(), wgb.C.c_size_t()
            wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_start(wgb.C.byref(start), table), "entry_start")
            wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_count(wgb.C.byref(count), table), "entry_count")
            lo, hi = start.value, start.value + count.value
            tu.scatter(torch.from_numpy(full[lo:hi]).cuda().to(tdt), torch.arange(lo, hi, device="cuda", dtype=torch.int64),
                       table, env)
            torch.cuda.synchronize()
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            want_all = to_host(torch.from_numpy(full).to(tdt))
            for step in range(5):
                rng = np.random.default_rng(100 * step + rank)
                n = 2_000 + 300 * rank
                ids = np.where(rng.random(n) < 0.8, rng.integers(0, rows // 10, size=n), rng.integers(0, rows, size=n))
                ids = ids.astype(np.int64)
                d_ids = torch.from_numpy(ids).cuda()
                out = torch.zeros((n, dim), dtype=tdt, device="cuda")
                wi, wo = tu.wrap_torch_tensor(d_ids), tu.wrap_torch_tensor(out)
                wgb.EmbeddingGatherForward(emb, wi, wo, step != 2, env, tu.current_stream_int())
                torch.cuda.synchronize()
                wgb.destroy_wholegraph_tensor(wi)
                wgb.destroy_wholegraph_tensor(wo)
                assert np.array_equal(to_host(out), want_all[ids]), f"node-level cached gather {step} differs on rank {rank}"
                wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            # something must have been cached: read all tag sets through the library (the tags live on the
            # cache communicator; a small shard may sit in a page of a neighbour's GPU, where torch cannot
            # wrap the pointer, but every rank of that communicator can gather from it)
            tags = wgb.embedding_cache_tensors(emb)[0]
            sets = wgb.lib().wholegraph_tensor_get_tensor_description(tags).contents.sizes[0]
            all_tags = torch.zeros((sets, 32), dtype=torch.int16, device="cuda")
            tu.gather(tags, torch.arange(sets, device="cuda", dtype=torch.int64), all_tags, env)
            torch.cuda.synchronize()
            assert int((all_tags != 0).sum().item()) > 32, "nothing was cached"
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            wgb.destroy_embedding(emb)
            wgb.destroy_cache_policy(policy)
        wgb.destroy_communicator(half)

    def run_unequal():
        # A different request length on every rank, rank 0 far above and the others far below the
        # 16 MiB at which a pipelined NCCL exchange is cut into chunks, and one rank with nothing to
        # ask for: every rank must still issue matching collectives.
        lengths = [150_000] + [5_000 + 100 * r for r in range(1, world - 1)] + [0]
        check_gather(MT.MtDistributed, 400_003, 128, torch.float16, torch.float16, lengths, seed=7)
        check_gather(MT.MtDistributed, 400_003, 64, torch.float32, torch.float32, lengths[::-1], seed=8)
        check_scatter(MT.MtDistributed, 400_003, 128, torch.float32, torch.float16, [90_000] + [3_000] * (world - 1))
        check_gather(MT.MtContinuous, 50_000, 32, torch.float32, torch.float32, lengths, seed=9)

    def run_stated_size():
        # BASELINE configuration C3's table at its stated size: 100,000,000 x 128 fp16, CONTINUOUS /
        # DEVICE, so that shard boundaries fall inside 2 MiB pages and byte offsets pass 2^32.  The
        # table holds a closed form of (row, column) evaluated on the GPU; a sample of ids (both
        # ends of every shard among them) is checked against the same form evaluated on the host.
        rows, dim, n = 100_000_000, 128, 200_000
        def form(r, c, xp):
            return (((r * 131 + c * 7) % 2001 - 1000).astype(xp.float32) / 1000.0) if xp is np else \
                (((r * 131 + c * 7) % 2001 - 1000).to(torch.float32) / 1000.0)
        for mem in (MT.MtContinuous, MT.MtChunked):
            print(f"rank {rank}: stated-size gather {mem.name}", flush=True)
            t = wgb.create_wholegraph_tensor(wgb.make_description([rows, dim], DT.DtHalf), comm, mem, ML.MlDevice)
            start, count = wgb.C.c_size_t(), wgb.C.c_size_t()
            wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_start(wgb.C.byref(start), t), "entry_start")
            wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_count(wgb.C.byref(count), t), "entry_count")
            cols = torch.arange(dim, device="cuda", dtype=torch.int64)[None, :]
            for s0 in range(0, count.value, 2_000_000):
                m = min(2_000_000, count.value - s0)
                r = torch.arange(start.value + s0, start.value + s0 + m, device="cuda", dtype=torch.int64)[:, None]
                tu.write_local_shard(t, form(r, cols, torch).to(torch.float16).contiguous(), s0)
            torch.cuda.synchronize()
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            off = orc.equal_partition_offsets(rows, world)
            ids = np.random.default_rng(50 + rank).integers(0, rows, size=n).astype(np.int64)
            edges = np.concatenate([off[:-1], off[1:] - 1, off[1:-1] - 1, [0, rows - 1]])
            ids[:len(edges)] = edges
            out = torch.zeros((n, dim), dtype=torch.float16, device="cuda")
            tu.gather(t, torch.from_numpy(ids).cuda(), out, env)
            torch.cuda.synchronize()
            want = form(ids[:, None], np.arange(dim, dtype=np.int64)[None, :], np).astype(np.float16)
            assert np.array_equal(out.cpu().numpy().view(np.int16), want.view(np.int16)), \
                f"stated-size gather {mem.name} differs on rank {rank}"
            # scatter rows all over the table (ids unique across ranks: congruent to the rank) and read them back
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            mine = (np.random.default_rng(3).permutation(rows // world)[:5_000].astype(np.int64) * world + rank)
            mine[:2] = [rank, (rows // world - 1) * world + rank]
            mine = np.unique(mine)
            vals = np.random.default_rng(60 + rank).uniform(-1, 1, size=(len(mine), dim)).astype(np.float16)
            d_mine = torch.from_numpy(mine).cuda()
            tu.scatter(torch.from_numpy(vals).cuda(), d_mine, t, env)
            torch.cuda.synchronize()
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            back = torch.zeros((len(mine), dim), dtype=torch.float16, device="cuda")
            tu.gather(t, d_mine, back, env)
            torch.cuda.synchronize()
            assert np.array_equal(back.cpu().numpy().view(np.int16), vals.view(np.int16)), \
                f"stated-size scatter {mem.name} differs on rank {rank}"
            wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
            wgb.destroy_wholegraph_tensor(t)

    def run_roundrobin():
        # Embedding with round_robin_size != 0 over several ranks: the literal remap of the reference
        # (map_indices_func.cu:16-34) adds the CALLER's first row, so a gather of id i on rank r
        # returns row entry_start(r) + rr * (block / world) + i % rr.
        rr, dim, rows = 8, 16, 8 * world * 20
        emb = wgb.create_embedding(wgb.make_description([rows, dim], DT.DtFloat), comm, MT.MtDistributed, ML.MlDevice,
                                   round_robin_size=rr)
        table = wgb.embedding_tensor(emb)
        full = table_values(rows, dim, np.float32)
        off = orc.equal_partition_offsets(rows, world)
        lo, hi = int(off[rank]), int(off[rank + 1])
        tu.scatter(torch.from_numpy(full[lo:hi]).cuda(), torch.arange(lo, hi, device="cuda", dtype=torch.int64), table, env)
        torch.cuda.synchronize()
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        ids = np.random.default_rng(rank).integers(0, rows, size=1_000).astype(np.int64)
        out = torch.zeros((len(ids), dim), dtype=torch.float32, device="cuda")
        d_ids = torch.from_numpy(ids).cuda()
        wi, wo = tu.wrap_torch_tensor(d_ids), tu.wrap_torch_tensor(out)
        wgb.EmbeddingGatherForward(emb, wi, wo, False, env, tu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wo)
        mapped = orc.round_robin_map(ids, rr=rr, world=world, entry_start=lo)
        assert np.array_equal(out.cpu().numpy(), full[mapped]), f"round-robin gather differs on rank {rank}"
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        wgb.destroy_embedding(emb)

    runners = {
        "fileio": run_fileio, "cache": run_cache, "optimizer": run_optimizer, "unequal": run_unequal,
        "stated-size": run_stated_size, "roundrobin": run_roundrobin, "hosttable": run_hosttable, "nodecache": run_nodecache,
        "continuous": lambda: run_memory_type(MT.MtContinuous),
        "distributed": lambda: run_memory_type(MT.MtDistributed),
        "chunked": lambda: run_memory_type(MT.MtChunked),
    }
    # A suffix selects one of the library's tuning switches for that scenario; the variables are
    # read again by a collective call, so one set of processes can run every variant in turn.
    switches = {"keepdups": {"WG_GATHER_DEDUP": "0"}, "nopresum": {"WG_GRADIENT_PRESUM": "0"},
                "peerpush": {"WG_PEER_GRADIENT": "1"}, "nccl": {"WG_PEER_EXCHANGE": "0"},
                "hostcounts": {"WG_SYNC_FREE": "0"}, "registers": {"WG_SERVE_BULK": "0"}}
    inherited = {k: os.environ.get(k) for sw in switches.values() for k in sw}
    for scenario in scenarios:
        base, suffix = scenario, ""
        parts = scenario.rsplit("-", 1)
        if len(parts) == 2 and parts[1] in switches:
            base, suffix = parts
        for k, v in inherited.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        os.environ.update(switches.get(suffix, {}))
        wgb.check(wgb.lib().wholegraph_b200_reload_tuning(comm), "reload_tuning")
        t0 = time.time()
        runners[base]()
        torch.cuda.synchronize()
        wgb.check(wgb.lib().wholegraph_communicator_barrier(comm), "barrier")
        print(f"rank {rank}: scenario {scenario} ok in {time.time() - t0:.1f} s", flush=True)
    wgb.destroy_communicator(comm)
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
