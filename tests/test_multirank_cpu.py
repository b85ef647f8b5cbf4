"""The distributed gather / gradient-routing protocol on CPU ranks (gloo, world_size 2 and 3).

Each rank runs the host logic of the DISTRIBUTED path with the oracle standing in for the
kernels: partition the request list by owner, exchange counts, exchange ids, then the W-step
ring in which a rank serves the rows its s-th neighbour asked for while receiving its own rows
from the (-s)-th neighbour, and finally the reorder.  The result must equal a plain gather on
the whole table, and the ring must not deadlock."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _table(rows, dim):
    return np.random.default_rng(0).uniform(-1, 1, size=(rows, dim)).astype(np.float32)


def _worker(rank, world, port, rows, dim, n, result_dir):
    sys.path.insert(0, ROOT)
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        off = orc.equal_partition_offsets(rows, world)
        table = _table(rows, dim)
        shard = table[off[rank]:off[rank + 1]]
        req = np.random.default_rng(100 + rank).integers(-2, rows, size=n).astype(np.int64)
        counts, sorted_ids, raw_pos = orc.bucket_sort_ids(req, off)
        send_counts = torch.from_numpy(counts.copy())
        recv_counts = torch.zeros(world, dtype=torch.int64)
        dist.all_to_all_single(recv_counts, send_counts)                       # counts exchange
        send_displs = np.concatenate([[0], np.cumsum(counts)[:-1]])
        recv_displs = np.concatenate([[0], np.cumsum(recv_counts.numpy())[:-1]])
        total_send, total_recv = int(counts.sum()), int(recv_counts.sum())
        recv_ids = torch.zeros(total_recv, dtype=torch.int64)
        dist.all_to_all_single(recv_ids, torch.from_numpy(sorted_ids[:total_send].copy()),
                               output_split_sizes=recv_counts.tolist(), input_split_sizes=counts.tolist())
        recv_ids = recv_ids.numpy()
        assert np.all((recv_ids >= off[rank]) & (recv_ids < off[rank + 1]))      # only rows this rank owns

        out = np.full((n, dim), 7, dtype=np.float16)
        # step 0: own rows straight to their output positions
        s0 = slice(int(send_displs[rank]), int(send_displs[rank] + counts[rank]))
        orc.gather(shard, sorted_ids[s0] - off[rank], out_dt=orc.DT_HALF, out=out, raw_pos=raw_pos[s0])
        recv_rows = np.zeros((total_send, dim), dtype=np.float16)
        for s in range(1, world):
            to, frm = (rank + s) % world, (rank - s) % world
            seg = slice(int(recv_displs[to]), int(recv_displs[to] + recv_counts[to]))
            served = orc.gather(shard, recv_ids[seg] - off[rank], out_dt=orc.DT_HALF)   # cast at the owner
            mine = slice(int(send_displs[frm]), int(send_displs[frm] + counts[frm]))
            ops = []
            if served.shape[0] > 0:
                ops.append(dist.isend(torch.from_numpy(served.view(np.int16)), to))
            buf = torch.zeros((int(counts[frm]), dim), dtype=torch.int16)
            if counts[frm] > 0:
                ops.append(dist.irecv(buf, frm))
            for op in ops:
                op.wait()
            recv_rows[mine] = buf.numpy().view(np.float16)
            out[raw_pos[mine]] = recv_rows[mine]                                         # reorder
        want = np.full((n, dim), 7, dtype=np.float16)
        orc.gather(table, req, out_dt=orc.DT_HALF, out=want)
        assert np.array_equal(out, want)
        with open(os.path.join(result_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_distributed_gather_protocol_on_gloo(tmp_path, world):
    port = 29600 + world + (os.getpid() % 200)
    mp.spawn(_worker, args=(world, port, 5_003, 8, 2_000, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def _chunked_worker(rank, world, port, rows, dim, ns, result_dir):
    """The chunked row exchange of a distributed scatter with a different request length on every
    rank: K comes from the library's rule on the all-gathered count matrix, every chunk is one
    matched round of sends and receives cut by the rule rows [c*k/K, c*(k+1)/K)."""
    import ctypes as C
    sys.path.insert(0, ROOT)
    from oracle import oracle as orc
    from __graft_entry__ import load_package
    wgb = load_package().binding
    wgb.load_library()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = ns[rank]
        off = orc.equal_partition_offsets(rows, world)
        req = np.random.default_rng(200 + rank).permutation(rows)[:n].astype(np.int64)   # unique ids
        rows_in = np.random.default_rng(300 + rank).integers(0, 1 << 15, size=(n, dim)).astype(np.int16)
        counts, sorted_ids, raw_pos = orc.bucket_sort_ids(req, off)
        gathered = [torch.zeros(world, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts.copy()))
        matrix = np.stack([g.numpy() for g in gathered])                                  # same on every rank
        row_bytes = dim * 2
        m = np.ascontiguousarray(matrix)
        K = wgb.lib().wholegraph_b200_exchange_chunk_count(m.ctypes.data_as(C.POINTER(C.c_int64)), world, row_bytes, 0, 0)
        ks = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(ks, torch.tensor([K], dtype=torch.int64))
        assert len({int(k) for k in ks}) == 1, "ranks disagree on the number of chunks"
        # the per-rank rule this replaces gives different answers for this matrix
        own_rule = 1 if (counts.sum() - counts[rank]) * row_bytes < (16 << 20) else 4
        rules = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(rules, torch.tensor([own_rule], dtype=torch.int64))
        assert len({int(k) for k in rules}) > 1, "the case does not straddle the threshold"

        send_displs = np.concatenate([[0], np.cumsum(counts)[:-1]])
        recv_counts = matrix[:, rank]
        recv_displs = np.concatenate([[0], np.cumsum(recv_counts)[:-1]])
        packed = rows_in[raw_pos[:int(counts.sum())]]
        recv_rows = np.zeros((int(recv_counts.sum()), dim), dtype=np.int16)
        recv_ids = np.zeros(int(recv_counts.sum()), dtype=np.int64)
        cut = lambda c, k: (c * k // K, c * (k + 1) // K)
        for k in range(K):
            ops, bufs = [], []
            for step in range(1, world):
                to, frm = (rank + step) % world, (rank - step) % world
                b, e = cut(int(counts[to]), k)
                if e > b:
                    lo = int(send_displs[to])
                    ops.append(dist.isend(torch.from_numpy(packed[lo + b:lo + e].copy()), to, tag=k))
                    ops.append(dist.isend(torch.from_numpy(sorted_ids[lo + b:lo + e].copy()), to, tag=100 + k))
                b, e = cut(int(recv_counts[frm]), k)
                if e > b:
                    rbuf = torch.zeros((e - b, dim), dtype=torch.int16)
                    ibuf = torch.zeros(e - b, dtype=torch.int64)
                    ops.append(dist.irecv(rbuf, frm, tag=k))
                    ops.append(dist.irecv(ibuf, frm, tag=100 + k))
                    bufs.append((int(recv_displs[frm]) + b, rbuf, ibuf))
            for op in ops:
                op.wait()
            for lo, rbuf, ibuf in bufs:
                recv_rows[lo:lo + rbuf.shape[0]] = rbuf.numpy()
                recv_ids[lo:lo + rbuf.shape[0]] = ibuf.numpy()
        lo = int(recv_displs[rank])
        me = slice(int(send_displs[rank]), int(send_displs[rank] + counts[rank]))
        recv_rows[lo:lo + int(counts[rank])] = packed[me]
        recv_ids[lo:lo + int(counts[rank])] = sorted_ids[me]
        # every row this rank owns that anybody scattered has arrived, with its id
        all_req = [np.random.default_rng(200 + q).permutation(rows)[:ns[q]].astype(np.int64) for q in range(world)]
        all_rows = [np.random.default_rng(300 + q).integers(0, 1 << 15, size=(ns[q], dim)).astype(np.int16) for q in range(world)]
        want = {}
        for q in range(world):
            mine = (all_req[q] >= off[rank]) & (all_req[q] < off[rank + 1])
            for i, r in zip(all_req[q][mine], all_rows[q][mine]):
                want[(q, int(i))] = r
        got = 0
        for q in range(world):
            seg = slice(int(recv_displs[q]), int(recv_displs[q] + recv_counts[q]))
            for i, r in zip(recv_ids[seg], recv_rows[seg]):
                assert np.array_equal(want[(q, int(i))], r)
                got += 1
        assert got == len(want)
        with open(os.path.join(result_dir, f"ok{rank}"), "w") as f:
            f.write(str(K))
    finally:
        dist.destroy_process_group()


def test_chunked_exchange_with_unequal_request_lengths_on_gloo(tmp_path):
    """Rank 0 scatters 40x as many rows as rank 1: rank 0 is above the 16 MiB threshold, rank 1
    far below it.  With the chunk count taken from the shared count matrix both run 4 matched
    rounds and every row arrives."""
    world, dim = 2, 512
    ns = [40_000, 1_000]           # 40,000 x 1 KiB rows: ~20 MB leave rank 0, ~0.5 MB leave rank 1
    port = 29650 + (os.getpid() % 200)
    mp.spawn(_chunked_worker, args=(world, port, 50_021, dim, ns, str(tmp_path)), nprocs=world, join=True)
    assert [(tmp_path / f"ok{r}").read_text() for r in range(world)] == ["4", "4"]


def test_bench_request_lists_are_seeded_and_in_range():
    """The benchmark's bounded power-law ranks: deterministic per seed, inside the table, skewed."""
    sys.path.insert(0, ROOT)
    rows, n, alpha = 1_000_000, 100_000, 1.1
    e = 1.0 - alpha

    def ranks(seed):
        u = np.random.default_rng(seed).random(n)
        return np.clip(np.floor(((rows ** e - 1.0) * u + 1.0) ** (1.0 / e)).astype(np.int64), 1, rows) - 1

    a, b = ranks(100), ranks(100)
    assert np.array_equal(a, b) and a.min() >= 0 and a.max() < rows
    assert not np.array_equal(a, ranks(101))
    assert (a == 0).mean() > 0.05 and np.unique(a).size < 0.8 * n   # heavy head, many duplicates
