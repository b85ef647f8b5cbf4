"""Benchmark of the WholeGraph gather hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One step = one wholegraph_gather call over one batch of synthetic, seeded indices.
  N = 1 : "C2"  table 10,000,000 x 128 fp32 (CONTINUOUS/DEVICE), 1,048,576 int64 ids uniform with
          replacement, output cast to fp16.
  N > 1 : "C3"  table 100,000,000 x 128 fp16 row-sharded CONTINUOUS/DEVICE (direct NVLink loads),
          1,048,576 int64 Zipf(1.1) ids per rank over a seeded permutation, fp16 output, every
          rank gathering at once (launch with torchrun, one rank per GPU).
Rank 0 prints one JSON line: `value` is gathered (output) GB/s summed over ranks with inputs
resident in HBM; `e2e` is the same metric with pinned-host index and output buffers copied
inside the timed region; `roofline` relates the copy kernel to the measured HBM (N = 1) or
NVLink (N > 1) peak; `cpu_baseline` times the CPU oracle on the host cores beside it.
`--impl reference` times only that CPU restatement (the reference has no CPU gather of its own).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROW_DIM = 128
IDS_PER_RANK = 1_048_576
HBM_FALLBACK_GBS = 6650.0   # earlier measurement on this pool, used only without MEASURED_PEAKS.json
NVLINK_PEER_GBS = 770.0     # measured peer copy, per direction per GPU
INDEX_BATCHES = 4           # distinct index batches cycled through the steps


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "c2", "c3", "c4", "c5", "cache", "unique"])
    ap.add_argument("--rows", type=int, default=0, help="override the table rows (profiling on a small case)")
    ap.add_argument("--ids", type=int, default=0, help="override the ids per rank")
    ap.add_argument("--env-sweep", default="",
                    help="gather workloads: time the steps once per setting of the library's tuning variables, e.g. "
                         "'WG_GATHER_DEDUP=1,WG_PEER_EXCHANGE=1;WG_GATHER_DEDUP=1,WG_PEER_EXCHANGE=0', one JSON line "
                         "per setting (same value on every rank), instead of the bench line")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val == "Active":
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}
        return out


def zipf_ids(torch, n, rows, alpha, perm, gen, shift=0.0):
    """Bounded power-law ranks P(k) ~ (k + shift)^-alpha by inverse CDF, mapped through a permutation
    of the row ids.  shift = 0 is a plain bounded Zipf; a positive shift (Zipf-Mandelbrot) flattens
    the head and is how a stated duplicate rate is met."""
    u = torch.rand(n, generator=gen, device="cuda", dtype=torch.float64)
    e = 1.0 - alpha
    lo, hi = (1.0 + shift) ** e, (float(rows) + shift) ** e
    rank = torch.floor(((hi - lo) * u + lo) ** (1.0 / e) - shift).to(torch.int64)
    rank = rank.clamp_(1, rows) - 1
    return perm[rank] if perm is not None else rank


def cpu_oracle_gather_rate(table_np, idx_np, out_dt, threads, budget_s=12.0, min_reps=2):
    """Output GB/s of the CPU oracle's gather on the host cores."""
    from oracle import oracle as orc
    import numpy as np
    n, dim = idx_np.shape[0], table_np.shape[1]
    out = np.zeros((n, dim), dtype=orc.np_dtype(out_dt))
    orc.gather(table_np, idx_np, out_dt=out_dt, out=out, threads=threads)  # warm-up
    times, t_begin = [], time.perf_counter()
    while len(times) < min_reps or (time.perf_counter() - t_begin < budget_s and len(times) < 40):
        t0 = time.perf_counter()
        orc.gather(table_np, idx_np, out_dt=out_dt, out=out, threads=threads)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return n * dim * out.itemsize / best / 1e9, best, len(times)


def run_reference_arm(args):
    """CPU restatement of the reference's gather on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import numpy as np
    from oracle import oracle as orc
    multi = args.gpus > 1
    threads = os.cpu_count() or 1
    ids = args.ids or IDS_PER_RANK
    # Bounded sample: the table is cut to what the host can fill in seconds; the request list
    # keeps its full length and its distribution.
    rows = args.rows or 2_000_000
    rng = np.random.default_rng(0)
    if multi:
        table = rng.uniform(-1, 1, size=(rows, ROW_DIM)).astype(np.float16)
        e = 1.0 - 1.1
        u = np.random.default_rng(100).random(ids)
        rank = np.clip(np.floor(((rows ** e - 1.0) * u + 1.0) ** (1.0 / e)).astype(np.int64), 1, rows) - 1
        idx = np.random.default_rng(7).permutation(rows)[rank]
        out_dt, workload = orc.DT_HALF, "C3 sample"
    else:
        table = rng.uniform(-1, 1, size=(rows, ROW_DIM)).astype(np.float32)
        idx = np.random.default_rng(1).integers(0, rows, size=ids, dtype=np.int64)
        out_dt, workload = orc.DT_HALF, "C2 sample"
    out = np.zeros((ids, ROW_DIM), dtype=orc.np_dtype(out_dt))
    for _ in range(max(args.warmup, 1)):
        orc.gather(table, idx, out_dt=out_dt, out=out, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.gather(table, idx, out_dt=out_dt, out=out, threads=threads)
    dt = time.perf_counter() - t0
    value = args.steps * ids * ROW_DIM * out.itemsize / dt / 1e9
    sample = f"{workload}: table cut to {rows} x {ROW_DIM} rows on the host, {ids} ids per step, {threads} threads"
    line = {
        "impl": "reference", "metric": "gathered embedding GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32->f16" if not multi else "f16", "data": "synthetic",
        "config": {"workload": workload, "note": "CPU restatement of the reference kernels (the reference has no CPU gather)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_sparse_adam(args, torch, dist, wgb, tu, comm, world, rank, local_rank):
    """C5: one Lazy Adam step per bench step on a DISTRIBUTED fp32 table of dim 256; every rank
    feeds 2,097,152 fp32 gradient rows at Zipf(1.1) ids; duplicates are summed before the update."""
    import ctypes as C
    dim, multi = 256, world > 1
    rows = args.rows or (50_000_000 if world == 8 else 6_250_000 * world)   # 6.25 M rows per GPU
    n = args.ids or 2_097_152
    DT, MT, ML = wgb.WholeGraphDataType, wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation
    env = wgb.cached_env_fns()
    emb = wgb.create_embedding(wgb.make_description([rows, dim], DT.DtFloat), comm, MT.MtDistributed, ML.MlDevice)
    opt = wgb.create_optimizer(wgb.WholeGraphOptimizerType.OptLazyAdam)
    wgb.check(wgb.lib().wholegraph_embedding_set_optimizer(emb, opt), "set_optimizer")
    table = wgb.embedding_tensor(emb)
    local_rows = C.c_size_t()
    wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_count(C.byref(local_rows), table), "entry_count")
    gen = torch.Generator(device="cuda").manual_seed(rank)
    for s in range(0, local_rows.value, 2_000_000):
        piece = torch.empty((min(2_000_000, local_rows.value - s), dim), dtype=torch.float32, device="cuda")
        piece.normal_(0, 0.01, generator=gen)
        tu.write_local_shard(table, piece, s)
    perm = torch.randperm(rows, generator=torch.Generator(device="cuda").manual_seed(7), device="cuda")
    batches = []
    for b in range(2):
        g = torch.Generator(device="cuda").manual_seed(1000 * b + rank)
        ids = zipf_ids(torch, n, rows, 1.1, perm, g)
        grads = torch.empty((n, dim), dtype=torch.float32, device="cuda").normal_(0, 1e-3, generator=g)
        batches.append((ids, grads, tu.wrap_torch_tensor(ids), tu.wrap_torch_tensor(grads)))
    del perm
    unique_global = int(torch.unique(batches[0][0]).numel())
    stream = tu.current_stream_int()

    def step(i):
        _, _, wi, wg = batches[i % 2]
        wgb.EmbeddingGatherGradientApply(emb, wi, wg, False, 1e-3, env, stream)

    def barrier():
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = wgb.lib().wholegraph_b200_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    launches = wgb.lib().wholegraph_b200_kernel_launch_count() - l0
    ms = e0.elapsed_time(e1)
    if multi:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        peak, how = measured_hbm_peak()
        # per rank: every raw gradient row read once (1024 B) + 7184 B per distinct row it owns
        alg = n * dim * 4 + (unique_global / world) * 7184 if not multi else n * dim * 4 + unique_global * 7184
        achieved = alg / (ms_step * 1e-3) / 1e9
        line = {"metric": "sparse-Adam rows/s", "value": world * n / (ms_step * 1e-3), "unit": "rows/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"C5: Lazy Adam on a {rows} x {dim} fp32 DISTRIBUTED table over {world} GPUs, "
                                       f"{n} gradient rows N(0,1e-3) per rank per step at Zipf(1.1) ids, lr 1e-3",
                           "distinct_ids_rank0_batch0": unique_global},
                "gpu_launches": int(launches), "clocks": clocks,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": None, "peak_source": how,
                             "note": "1024 B per raw gradient row + 7184 B per distinct updated row (single-rank estimate "
                                     "from rank 0's first batch)"}}
        print(json.dumps(line), flush=True)
    for _, _, wi, wg in batches:
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wg)
    barrier()
    wgb.destroy_embedding(emb)
    wgb.lib().wholegraph_destroy_embedding_optimizer(opt)
    wgb.destroy_communicator(comm)
    if multi:
        dist.destroy_process_group()


def run_cached_gather(args, torch, wgb, tu, comm):
    """Cached embedding gather on one GPU: a 10 M x 128 fp32 table behind a set-associative cache
    holding one row in eight (sets of 32 lines over 256 rows), 1,048,576 Zipf(1.1) ids per step
    over a seeded permutation, fp32 output.  Timed twice: lookups only (adjust_cache = False, after
    the cache has been warmed) and with the LFU update of every step inside the timed region."""
    import ctypes as C
    dim = ROW_DIM
    rows = args.rows or 10_000_000
    n = args.ids or IDS_PER_RANK
    DT, MT, ML, AT = (wgb.WholeGraphDataType, wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation,
                      wgb.WholeGraphAccessType)
    env = wgb.cached_env_fns()
    policy = wgb.create_cache_policy(comm, MT.MtContinuous, ML.MlDevice, AT.AtReadWrite, 0.125)
    emb = wgb.create_embedding(wgb.make_description([rows, dim], DT.DtFloat), comm, MT.MtContinuous, ML.MlDevice,
                               cache_policy=policy)
    table = wgb.embedding_tensor(emb)
    local_rows = C.c_size_t()
    wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_count(C.byref(local_rows), table), "entry_count")
    gen = torch.Generator(device="cuda").manual_seed(3)
    for s in range(0, local_rows.value, 2_000_000):
        piece = torch.empty((min(2_000_000, local_rows.value - s), dim), dtype=torch.float32, device="cuda")
        piece.uniform_(-1, 1, generator=gen)
        tu.write_local_shard(table, piece, s)
    perm = torch.randperm(rows, generator=torch.Generator(device="cuda").manual_seed(7), device="cuda")
    batches = [zipf_ids(torch, n, rows, 1.1, perm, torch.Generator(device="cuda").manual_seed(100 + b))
               for b in range(INDEX_BATCHES)]
    del perm
    wraps = [tu.wrap_torch_tensor(b) for b in batches]
    out = torch.empty((n, dim), dtype=torch.float32, device="cuda")
    wout = tu.wrap_torch_tensor(out)
    stream = tu.current_stream_int()

    def timed(adjust):
        for i in range(args.warmup):
            wgb.EmbeddingGatherForward(emb, wraps[i % INDEX_BATCHES], wout, adjust, env, stream)
        torch.cuda.synchronize()
        l0 = wgb.lib().wholegraph_b200_kernel_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            wgb.EmbeddingGatherForward(emb, wraps[i % INDEX_BATCHES], wout, adjust, env, stream)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps, wgb.lib().wholegraph_b200_kernel_launch_count() - l0

    for i in range(2 * INDEX_BATCHES):      # warm the cache with every batch
        wgb.EmbeddingGatherForward(emb, wraps[i % INDEX_BATCHES], wout, True, env, stream)
    sampler = ClockSampler(0)
    sampler.start()
    ms_lookup, launches = timed(False)
    ms_adjust, _ = timed(True)
    clocks = sampler.stop()
    tags = wgb.embedding_cache_tensors(emb)[0]
    sets = wgb.lib().wholegraph_tensor_get_tensor_description(tags).contents.sizes[0]
    peak, how = measured_hbm_peak()
    algorithmic = n * (2 * dim * 4 + 8 + 64)       # row read + row write + id + one 64-byte tag set per id
    achieved = algorithmic / (ms_lookup * 1e-3) / 1e9
    line = {"metric": "gathered embedding GB/s", "value": n * dim * 4 / (ms_lookup * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_lookup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cached gather: {rows} x {dim} fp32 CONTINUOUS/DEVICE table behind a cache of ratio 1/8 "
                                   f"({sets} sets of 32 lines), {n} int64 Zipf(1.1) ids per step, fp32 output, lookups only",
                       "ms_per_step_with_lfu_update": ms_adjust,
                       "value_with_lfu_update": n * dim * 4 / (ms_adjust * 1e-3) / 1e9},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": how, "algorithmic_bytes_per_launch": algorithmic,
                         "note": "row read + row written + id + one 64-byte tag set per id, no credit for repeats; the "
                                 "hot rows of a Zipf list and their tag sets are served from L2, so this can exceed 1"}}
    print(json.dumps(line), flush=True)
    for w in wraps:
        wgb.destroy_wholegraph_tensor(w)
    wgb.destroy_wholegraph_tensor(wout)
    wgb.destroy_embedding(emb)
    wgb.destroy_cache_policy(policy)


def run_append_unique(args, torch, wgb, tu):
    """graph_append_unique on one GPU with the shapes of the last hop of a [15, 10, 5] fan-out from 1,024
    seeds: 153,600 distinct int64 target nodes and 768,000 sampled neighbours (Zipf(1.2) over 240 M node ids,
    some of them targets).  A step is one call, output allocation and its two stream synchronisations
    included."""
    t_count, n_count, nodes = 153_600, args.ids or 768_000, args.rows or 240_000_000
    g = torch.Generator(device="cuda").manual_seed(11)
    perm_seed = torch.Generator(device="cuda").manual_seed(7)
    targets = torch.randperm(nodes, generator=perm_seed, device="cuda")[:t_count].contiguous()
    batches = []
    for b in range(INDEX_BATCHES):
        ids = zipf_ids(torch, n_count, nodes, 1.2, None, torch.Generator(device="cuda").manual_seed(50 + b), 1.4e5)
        ids[: n_count // 8] = targets[torch.randint(0, t_count, (n_count // 8,), generator=g, device="cuda")]
        batches.append(ids.contiguous())
    mapping = torch.empty(n_count, dtype=torch.int32, device="cuda")
    wt, wm = tu.wrap_torch_tensor(targets), tu.wrap_torch_tensor(mapping)
    wn = [tu.wrap_torch_tensor(b) for b in batches]
    env, stream = wgb.cached_env_fns(), tu.current_stream_int()
    slot = wgb.OutputSlot()

    def step(i):
        wgb.append_unique(wt, wn[i % INDEX_BATCHES], slot, wm, env, stream)
        n_unique = slot.description.sizes[0]
        wgb.release_output(slot)
        return n_unique

    for i in range(args.warmup):
        n_unique = step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    l0 = wgb.lib().wholegraph_b200_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        n_unique = step(i)
    e1.record()
    torch.cuda.synchronize()
    launches = wgb.lib().wholegraph_b200_kernel_launch_count() - l0
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    peak, how = measured_hbm_peak()
    m = t_count + n_count
    algorithmic = m * 8 + n_count * 4 + n_unique * 8      # ids read once, mapping and list written once
    achieved = algorithmic / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "append-unique nodes/s", "value": m / (ms * 1e-3), "unit": "nodes/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": {"workload": f"graph_append_unique: {t_count} distinct int64 targets + {n_count} neighbours "
                               f"(Zipf(1.2, shift 1.4e5) over {nodes} node ids, 1/8 of them targets), with mapping",
                   "unique_nodes_last_step": int(n_unique)},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": how, "algorithmic_bytes_per_launch": algorithmic,
                     "note": "ids read once, mapping and node list written once; the radix sort's passes and the "
                             "two host synchronisations are overhead, so this op is latency-bound at this size"}}),
          flush=True)
    for w in [wt, wm] + wn:
        wgb.destroy_wholegraph_tensor(w)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    pkg = load_package()
    wgb = pkg.binding
    from cugraph_gnn_b200 import torch_utils as tu
    wgb.load_library()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run, one rank per GPU")
    torch.cuda.set_device(local_rank)
    wgb.init(0, 2)
    multi = world > 1
    workload = args.workload if args.workload != "auto" else ("c3" if multi else "c2")

    comm = None
    if multi:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        raw = wgb.unique_id_to_bytes(wgb.create_unique_id()) if rank == 0 else bytes(128)
        buf = torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()
        dist.broadcast(buf, 0)
        uid = wgb.unique_id_from_bytes(buf.cpu().numpy().tobytes())
        comm = wgb.create_communicator(uid, rank, world)
    else:
        comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)

    if workload == "c5":
        run_sparse_adam(args, torch, dist, wgb, tu, comm, world, rank, local_rank)
        return
    if workload == "unique":
        if multi:
            raise SystemExit("the append-unique workload runs on one GPU")
        run_append_unique(args, torch, wgb, tu)
        return
    if workload == "cache":
        if multi:
            raise SystemExit("the cache workload runs on one GPU")
        run_cached_gather(args, torch, wgb, tu, comm)
        return
    MT = wgb.WholeGraphMemoryType
    mem_type, zipf_alpha, zipf_shift = MT.MtContinuous, None, 0.0
    if workload == "c2":
        n_ids = args.ids or IDS_PER_RANK
        rows = args.rows or 10_000_000
        tab_dtype, out_dtype, tab_wg = torch.float32, torch.float16, wgb.WholeGraphDataType.DtFloat
        name = f"C2: {rows} x {ROW_DIM} fp32 CONTINUOUS/DEVICE table, {n_ids} int64 ids uniform with replacement, gather with cast to fp16"
    elif workload == "c3":
        n_ids = args.ids or IDS_PER_RANK
        rows = args.rows or 100_000_000
        zipf_alpha = 1.1
        tab_dtype, out_dtype, tab_wg = torch.float16, torch.float16, wgb.WholeGraphDataType.DtHalf
        name = (f"C3: {rows} x {ROW_DIM} fp16 table row-sharded CONTINUOUS/DEVICE over {world} GPUs, "
                f"{n_ids} int64 Zipf(1.1) ids per rank over a seeded permutation, fp16 output")
    else:
        n_ids = args.ids or 4_194_304
        rows = args.rows or 240_000_000
        # Zipf-Mandelbrot shift calibrated so that a 4,194,304-id request over 240 M rows holds
        # about 30 % duplicates, the rate the configuration states.
        zipf_alpha, zipf_shift, mem_type = 1.2, 1.4e5, MT.MtDistributed
        tab_dtype, out_dtype, tab_wg = torch.bfloat16, torch.bfloat16, wgb.WholeGraphDataType.DtBF16
        name = (f"C4: {rows} x {ROW_DIM} bf16 table row-sharded DISTRIBUTED (NCCL exchange) over {world} GPUs, "
                f"{n_ids} int64 Zipf(1.2, shift 1.4e5: ~30% duplicates) ids per rank over a seeded permutation, bf16 output")
    es_tab = torch.empty((), dtype=tab_dtype).element_size()
    es_out = torch.empty((), dtype=out_dtype).element_size()

    desc = wgb.make_description([rows, ROW_DIM], tab_wg)
    table = wgb.create_wholegraph_tensor(desc, comm, mem_type, wgb.WholeGraphMemoryLocation.MlDevice)
    local_rows = wgb.C.c_size_t()
    wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_count(wgb.C.byref(local_rows), table), "entry_count")
    local_rows = local_rows.value
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    chunk = 4_000_000
    for s in range(0, local_rows, chunk):  # fill in pieces through the C ABI (raw shard pointer)
        rows_now = min(chunk, local_rows - s)
        piece = torch.empty((rows_now, ROW_DIM), dtype=torch.float32, device="cuda").uniform_(-1, 1, generator=gen)
        tu.write_local_shard(table, piece.to(tab_dtype).contiguous(), s)
        del piece
    torch.cuda.synchronize()

    batches = []
    if workload == "c2":
        for b in range(INDEX_BATCHES):
            g = torch.Generator(device="cuda").manual_seed(1 + b)
            batches.append(torch.randint(0, rows, (n_ids,), generator=g, device="cuda", dtype=torch.int64))
    else:
        perm = torch.randperm(rows, generator=torch.Generator(device="cuda").manual_seed(7), device="cuda")
        for b in range(INDEX_BATCHES):
            g = torch.Generator(device="cuda").manual_seed(100 + rank + 1000 * b)
            batches.append(zipf_ids(torch, n_ids, rows, zipf_alpha, perm, g, zipf_shift))
        del perm
        torch.cuda.empty_cache()
    out = torch.empty((n_ids, ROW_DIM), dtype=out_dtype, device="cuda")
    env = wgb.cached_env_fns()
    wraps = [tu.wrap_torch_tensor(b) for b in batches]
    wout = tu.wrap_torch_tensor(out)
    stream = tu.current_stream_int()

    def step(i):
        wgb.wholegraph_gather_op(table, wraps[i % INDEX_BATCHES], wout, env, stream)

    def barrier():
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if not multi:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.env_sweep:
        # Tuning sweep: the library reads its WG_* variables at every call, so one process can
        # compare settings on the same table and index batches.
        for setting in args.env_sweep.split(";"):
            pairs = dict(kv.split("=", 1) for kv in setting.split(",") if kv)
            os.environ.update(pairs)
            for i in range(args.warmup):
                step(i)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                step(i)
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
            if rank == 0:
                print(json.dumps({"variant": pairs, "workload": name, "n_gpus": world, "steps": args.steps,
                                  "ms_per_step": ms,
                                  "value": world * n_ids * ROW_DIM * es_out / (ms * 1e-3) / 1e9, "unit": "GB/s"}),
                      flush=True)
        return

    # ---- device-resident timing ------------------------------------------------------------
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = wgb.lib().wholegraph_b200_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    launches = wgb.lib().wholegraph_b200_kernel_launch_count() - launches0
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    out_bytes = n_ids * ROW_DIM * es_out
    value = world * out_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end: pinned host ids in, pinned host rows out, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        h_idx = [b.cpu().pin_memory() for b in batches]
        h_out = torch.empty((n_ids, ROW_DIM), dtype=out_dtype).pin_memory()
        d_idx = torch.empty_like(batches[0])
        w_didx = tu.wrap_torch_tensor(d_idx)

        def e2e_step(i):
            d_idx.copy_(h_idx[i % INDEX_BATCHES], non_blocking=True)
            wgb.wholegraph_gather_op(table, w_didx, wout, env, stream)
            h_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the caller reads the rows on the host

        for i in range(min(args.warmup, 3)):
            e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        barrier()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / args.steps
        e2e = {"value": world * out_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": n_ids * 8, "d2h_bytes_per_step": out_bytes,
               "ms_per_step": e2e_ms}
        wgb.destroy_wholegraph_tensor(w_didx)
    clocks = sampler.stop() if rank == 0 else None

    # ---- roofline of the copy kernel -------------------------------------------------------
    algorithmic = n_ids * (ROW_DIM * es_tab + ROW_DIM * es_out + 8)   # row read + row write + id read
    if multi:
        per = -(-rows // world)
        b0 = batches[0]
        remote = b0[(b0 // per) != rank]
        remote_ids, remote_unique = int(remote.numel()), int(torch.unique(remote).numel())
        wire_row = ROW_DIM * (es_out if workload == "c4" else es_tab)   # DISTRIBUTED casts at the owner
        ingress = remote_ids * wire_row
        achieved = ingress / (ms_step * 1e-3) / 1e9
        roofline = {"bound": "nvlink", "achieved": achieved, "peak": NVLINK_PEER_GBS, "unit": "GB/s",
                    "frac": achieved / NVLINK_PEER_GBS, "traffic": None,
                    "remote_ids": remote_ids, "remote_unique_ids": remote_unique,
                    "note": "NVLink ingress per rank per step = ids owned by other ranks x row bytes (rank 0, "
                            "batch 0), no credit for repeated ids, over the measured 770 GB/s peer copy (of "
                            "measured); on mapped memory repeated remote rows are served by caches, so a "
                            "skewed request list can exceed 1"}
    else:
        peak, how = measured_hbm_peak()
        achieved = algorithmic / (ms_step * 1e-3) / 1e9
        # DRAM bytes per launch from the ncu capture of this kernel on a 2 M-row table with the full
        # 1,048,576-id list (profiles/row_copy_gather_c2.md): 520.4 MB read + 228.4 MB written; it
        # grows with the ids processed, so it is scaled by them.
        traffic = 748.8e6 * n_ids / 1_048_576 if workload == "c2" and out_dtype == torch.float16 else None
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "traffic": traffic, "peak_source": how,
                    "algorithmic_bytes_per_launch": algorithmic,
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch, small-table "
                                      "capture scaled by ids" if traffic else None}

    # ---- CPU oracle beside it (rank 0, N = 1 only) ----------------------------------------
    cpu = None
    if not multi and not args.no_cpu_baseline and rank == 0:
        from oracle import oracle as orc
        sample_rows = min(rows, 2_000_000)
        sample_ids = torch.arange(sample_rows, device="cuda", dtype=torch.int64)
        sample = torch.empty((sample_rows, ROW_DIM), dtype=tab_dtype, device="cuda")
        tu.gather(table, sample_ids, sample, env)
        torch.cuda.synchronize()
        table_np = sample.cpu().numpy()
        del sample, sample_ids
        idx_np = (batches[0] % sample_rows).cpu().numpy()
        threads = os.cpu_count() or 1
        gbs, best, reps = cpu_oracle_gather_rate(table_np, idx_np, orc.DT_HALF, threads)
        cpu = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": f"first {sample_rows} table rows on the host, {n_ids} ids, best of {reps} passes "
                         f"({best * 1e3:.1f} ms) of the CPU oracle's gather with cast to fp16"}

    if rank == 0:
        line = {
            "metric": "gathered embedding GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"c2": "f32->f16", "c3": "f16", "c4": "bf16"}[workload], "data": "synthetic",
            "config": {"workload": name, "l2": "table and output larger than L2; a different index batch each step",
                       "memory_type": ("DISTRIBUTED" if workload == "c4" else "CONTINUOUS") + "/DEVICE", "ids_per_rank": n_ids, "rows": rows, "dim": ROW_DIM},
            "gpu_launches": int(launches), "roofline": roofline, "clocks": clocks,
        }
        if e2e is not None:
            line["e2e"] = e2e
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)

    for w in wraps + [wout]:
        wgb.destroy_wholegraph_tensor(w)
    barrier()
    wgb.destroy_wholegraph_tensor(table)
    wgb.destroy_communicator(comm)
    if multi:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
