"""Benchmark of the WholeGraph gather / scatter / sparse-optimizer hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One step = one pass of the hot path over one batch of synthetic, seeded input, through the C ABI.
  N = 1 : "C2"  table 10,000,000 x 128 fp32 (CONTINUOUS/DEVICE), 1,048,576 int64 ids uniform with
          replacement, gather with the output cast to fp16.
  N > 1 : "C3"  table 100,000,000 x 128 fp16 row-sharded CONTINUOUS/DEVICE (direct NVLink loads),
          1,048,576 int64 Zipf(1.1) ids per rank over a seeded permutation, fp16 output, every
          rank gathering at once (launch with torchrun, one rank per GPU).
Rank 0 prints ONE JSON line.  `value` is gathered (output) GB/s summed over ranks with inputs
resident in HBM; `e2e` is the same metric with pinned-host index and output buffers copied inside
the timed region; `roofline` relates the copy kernel to the measured HBM (N = 1) or NVLink (N > 1)
peak; `parity` compares sampled output rows bit for bit with the table rows regenerated from the
fill seed (and cast by the CPU oracle); `cpu_baseline` times the CPU oracle on the host cores
beside it.  `extra` holds the other configurations of the metric, each timed for about a second
with its own clock record and parity check:
  N = 1 : scatter (C2: 1,048,576 unique-id fp16 rows into the fp32 table), c5 (sparse Lazy Adam
          rows/s), ref_gpu_kernel (the reference's own CUDA kernels on the same inputs, when the
          cross-check library was built).
  N > 1 : c3_unique (duplicate-free request lists: every remote row crosses NVLink),
          c3_single_gpu (the C3 shape with all rows local), d2h_floor (concurrent pinned
          device-to-host copies, what bounds e2e), c4 (DISTRIBUTED gather, bf16), c5 (sparse Lazy Adam
          over all ranks).
`--workload c2|c3|c3-unique|c4|c5|cache|unique` prints the line of one configuration instead.
`--impl reference` times the CPU restatement of the reference's gather on the host cores (the
reference has no CPU gather of its own).  A parity mismatch makes the run exit non-zero.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROW_DIM = 128
IDS_PER_RANK = 1_048_576
HBM_FALLBACK_GBS = 6650.0   # earlier measurement on this pool, used only without MEASURED_PEAKS.json
NVLINK_PEER_GBS = 770.0     # peer copy measured on this pool, per direction per GPU (nominal 900)
NVLINK_NOMINAL_GBS = 900.0
INDEX_BATCHES = 4           # distinct index batches cycled through the steps
FILL_CHUNK = 4_000_000      # table rows generated per piece (part of the fill's definition: the
                            # parity check regenerates rows with the same sequence of draws)
PARITY_SAMPLE = 4096        # output rows checked per rank


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="auto",
                    choices=["auto", "c2", "c3", "c3-unique", "c4", "c5", "cache", "unique", "p2p"])
    ap.add_argument("--rows", type=int, default=0, help="override the table rows (profiling on a small case)")
    ap.add_argument("--ids", type=int, default=0, help="override the ids per rank")
    ap.add_argument("--env-sweep", default="",
                    help="gather workloads: time the steps once per setting of the library's tuning variables, e.g. "
                         "'WG_GATHER_DEDUP=1,WG_PEER_EXCHANGE=1;WG_GATHER_DEDUP=1,WG_PEER_EXCHANGE=0', one JSON line "
                         "per setting (same value on every rank), instead of the bench line")
    ap.add_argument("--extra-seconds", type=float, default=1.0, help="timed seconds of each extra configuration")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    return ap.parse_args()


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


# ---- clocks --------------------------------------------------------------------------------
class ClockMonitor:
    """SM clock and throttle reasons of one GPU, sampled every 10 ms through NVML (read-only) by
    a thread of this process for as long as the benchmark runs; a leg asks for the summary of
    the samples that fell into its timed region.  Falls back to an nvidia-smi loop when NVML
    cannot be loaded."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, torch, device_index: int):
        self.samples = []          # (time.time(), sm MHz, reason bit mask)
        self.max_mhz = None
        self.handle = None
        self.nvml = None
        self.lock = threading.Lock()
        self.stop_flag = False
        self.thread = None
        self.proc = None
        try:
            import pynvml
            pynvml.nvmlInit()
            props = torch.cuda.get_device_properties(device_index)
            try:
                bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
                self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
                ids = [v for v in visible.split(",") if v.strip().isdigit()]
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(int(ids[device_index]) if ids else device_index)
            self.nvml = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:
            self.nvml = None
            self._start_smi(device_index)

    def _sample(self):
        try:
            sm = float(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
            mask = int(self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
            with self.lock:
                self.samples.append((time.time(), sm, mask))
        except Exception:
            pass

    def _loop(self):
        while not self.stop_flag:
            self._sample()
            time.sleep(0.01)

    def _start_smi(self, device_index):
        try:
            self.smi_file = open(os.path.join("/tmp", f"wg_bench_clocks_{os.getpid()}.csv"), "w+")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(device_index),
                 "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.smi_file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def begin(self):
        if self.nvml is not None:
            self._sample()
        elif self.proc is not None:
            self.smi_file.flush()
            return ("smi", os.path.getsize(self.smi_file.name))
        return ("t", time.time())

    def end(self, mark):
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        if self.nvml is not None:
            self._sample()
            with self.lock:
                got = [s for s in self.samples if s[0] >= mark[1]]
            if got:
                mask = 0
                for s in got:
                    mask |= s[2]
                out.update(sm_mhz=statistics.median(s[1] for s in got), samples=len(got),
                           reasons=[name for name, bit in self.REASONS if mask & bit])
            return out
        if self.proc is None:
            return out
        time.sleep(0.12)
        self.smi_file.flush()
        with open(self.smi_file.name) as f:
            f.seek(mark[1])
            lines = f.read().splitlines()
        sm, mx, reasons = [], [], set()
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for (name, _), val in zip(self.REASONS, parts[2:6]):
                if val == "Active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out

    def close(self):
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            try:
                os.unlink(self.smi_file.name)
            except OSError:
                pass


def bind_to_gpu_local_cpus(torch, device_index):
    """Restrict this process to the CPU cores next to its GPU before it allocates pinned host
    buffers, so that they land in the memory of the GPU's own NUMA node.  Returns what was done."""
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/local_cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        usable = cpus & os.sched_getaffinity(0)
        if not usable:
            return "gpu-local cpu list not usable from this process"
        os.sched_setaffinity(0, usable)
        return f"process bound to the {len(usable)} cores local to its GPU ({text})"
    except Exception as exc:  # no sysfs entry, no permission: leave the process as it is
        return f"not bound ({type(exc).__name__})"


# ---- synthetic inputs ------------------------------------------------------------------------
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


def equal_first_rows(rows, world):
    per = -(-rows // world)
    return [min(r * per, rows) for r in range(world + 1)]


def fill_shard(torch, tu, table, local_rows, dim, tab_dtype, seed):
    """This rank's shard: uniform(-1, 1) fp32 draws from a seeded generator, FILL_CHUNK rows per
    draw, cast to the table dtype, written through the C ABI."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    for s in range(0, local_rows, FILL_CHUNK):
        rows_now = min(FILL_CHUNK, local_rows - s)
        piece = torch.empty((rows_now, dim), dtype=torch.float32, device="cuda").uniform_(-1, 1, generator=gen)
        tu.write_local_shard(table, piece.to(tab_dtype).contiguous(), s)
        del piece
    torch.cuda.synchronize()


def regenerate_rows(torch, ids, first_row, dim, tab_dtype, seed_of_owner):
    """Rows `ids` (global, on the GPU) of a table filled by fill_shard on every owner, rebuilt from
    the owners' seeds without reading the table.  Ids nobody owns give zero rows."""
    out = torch.zeros((ids.numel(), dim), dtype=tab_dtype, device="cuda")
    for owner in range(len(first_row) - 1):
        lo, hi = first_row[owner], first_row[owner + 1]
        mine = (ids >= lo) & (ids < hi)
        if not bool(mine.any()):
            continue
        last_needed = int(ids[mine].max().item()) - lo
        gen = torch.Generator(device="cuda").manual_seed(seed_of_owner(owner))
        for s in range(0, hi - lo, FILL_CHUNK):
            rows_now = min(FILL_CHUNK, hi - lo - s)
            piece = torch.empty((rows_now, dim), dtype=torch.float32, device="cuda").uniform_(-1, 1, generator=gen)
            here = mine & (ids >= lo + s) & (ids < lo + s + rows_now)
            if bool(here.any()):
                out[here] = piece[ids[here] - lo - s].to(tab_dtype)
            del piece
            if s + rows_now > last_needed:
                break
    return out


def bits(torch, t):
    """Host integer view of a tensor's bit patterns."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).cpu().numpy()
    if t.dtype == torch.float32:
        return t.contiguous().view(torch.int32).cpu().numpy()
    return t.cpu().numpy()


# ---- CPU legs --------------------------------------------------------------------------------
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


def gather_config(workload, world, rows, n_ids):
    """The `config` object of a gather line; both arms print the same one."""
    if workload == "c2":
        name = (f"C2: {rows} x {ROW_DIM} fp32 CONTINUOUS/DEVICE table, {n_ids} int64 ids uniform with replacement, "
                f"gather with cast to fp16")
    elif workload == "c3":
        name = (f"C3: {rows} x {ROW_DIM} fp16 table row-sharded CONTINUOUS/DEVICE over {world} GPUs, "
                f"{n_ids} int64 Zipf(1.1) ids per rank over a seeded permutation, fp16 output")
    elif workload == "c3-unique":
        name = (f"C3 with duplicate-free request lists: {rows} x {ROW_DIM} fp16 table row-sharded CONTINUOUS/DEVICE over "
                f"{world} GPUs, {n_ids} distinct int64 ids per rank (slices of a seeded permutation), fp16 output")
    elif workload == "c3-single":
        name = (f"C3 shape on one GPU: {rows} x {ROW_DIM} fp16 CONTINUOUS/DEVICE table, all rows local, "
                f"{n_ids} int64 Zipf(1.1) ids over a seeded permutation, fp16 output")
    else:
        name = (f"C4: {rows} x {ROW_DIM} bf16 table row-sharded DISTRIBUTED over {world} GPUs, {n_ids} int64 "
                f"Zipf(1.2, shift 1.4e5: ~30% duplicates) ids per rank over a seeded permutation, bf16 output")
    return {"workload": name, "l2": "table and output larger than L2; a different index batch each step",
            "memory_type": ("DISTRIBUTED" if workload == "c4" else "CONTINUOUS") + "/DEVICE",
            "ids_per_rank": n_ids, "rows": rows, "dim": ROW_DIM}


def fill_host_table(np, rows, dim, dtype, threads):
    """uniform(-1, 1) rows on the host, drawn by `threads` workers over row ranges (numpy's
    generators release the interpreter lock)."""
    table = np.empty((rows, dim), dtype=dtype)
    piece = 262_144
    starts = list(range(0, rows, piece))

    def work(k):
        rng = np.random.default_rng(10_000 + k)
        for s in starts[k::threads]:
            e = min(rows, s + piece)
            block = rng.random((e - s, dim), dtype=np.float32)
            block *= 2.0
            block -= 1.0
            table[s:e] = block
    pool = [threading.Thread(target=work, args=(k,)) for k in range(threads)]
    for t in pool:
        t.start()
    for t in pool:
        t.join()
    return table


def run_reference_arm(args):
    """CPU restatement of the reference's gather on the host cores; rank 0 only.  The table has the
    configuration's full size when the host has the memory for it (it is cut, and the line says so,
    when it has not); a step is one rank's request list."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import numpy as np
    from oracle import oracle as orc
    multi = args.gpus > 1
    threads = os.cpu_count() or 1
    ids = args.ids or IDS_PER_RANK
    full_rows = 100_000_000 if multi else 10_000_000
    es = 2 if multi else 4
    rows = args.rows or full_rows
    note = None
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 8 << 30
    need = rows * ROW_DIM * es
    if need * 1.3 > avail:
        rows = max(1_000_000, int(avail * 0.5 / (ROW_DIM * es)) // 1_000_000 * 1_000_000)
        note = f"table cut to {rows} rows: the host has {avail / 2**30:.0f} GiB free"
    table = fill_host_table(np, rows, ROW_DIM, np.float16 if multi else np.float32, min(threads, 32))
    if multi:
        e = 1.0 - 1.1
        u = np.random.default_rng(100).random(ids)
        rank = np.clip(np.floor(((rows ** e - 1.0) * u + 1.0) ** (1.0 / e)).astype(np.int64), 1, rows) - 1
        idx = np.random.default_rng(7).permutation(rows)[rank]
        out_dt, workload = orc.DT_HALF, "c3"
    else:
        idx = np.random.default_rng(1).integers(0, rows, size=ids, dtype=np.int64)
        out_dt, workload = orc.DT_HALF, "c2"
    out = np.zeros((ids, ROW_DIM), dtype=orc.np_dtype(out_dt))
    for _ in range(max(args.warmup, 1)):
        orc.gather(table, idx, out_dt=out_dt, out=out, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.gather(table, idx, out_dt=out_dt, out=out, threads=threads)
    dt = time.perf_counter() - t0
    value = args.steps * ids * ROW_DIM * out.itemsize / dt / 1e9
    sample = (f"CPU restatement of the reference kernels (the reference has no CPU gather): {rows} x {ROW_DIM} table on "
              f"the host, one rank's list of {ids} ids per step, {threads} threads")
    config = gather_config(workload, max(args.gpus, 1), rows, ids)
    line = {
        "impl": "reference", "metric": "gathered embedding GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32->f16" if not multi else "f16", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if note:
        line["note"] = note
    print(json.dumps(line), flush=True)


# ---- shared run context ----------------------------------------------------------------------
class Context:
    def __init__(self, args, torch, dist, wgb, tu, comm, world, rank, local_rank):
        self.args, self.torch, self.dist, self.wgb, self.tu = args, torch, dist, wgb, tu
        self.comm, self.world, self.rank, self.local_rank = comm, world, rank, local_rank
        self.multi = world > 1
        self.env = wgb.cached_env_fns()
        self.monitor = ClockMonitor(torch, local_rank) if rank == 0 else None
        self.failures = []

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.multi:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if not self.multi:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def min_over_ranks(self, x):
        return -self.max_over_ranks(-x)

    def sum_over_ranks(self, x):
        if not self.multi:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def launches(self):
        return int(self.wgb.lib().wholegraph_b200_kernel_launch_count())

    def timed(self, step, steps, warmup):
        """`steps` back-to-back calls of step(i) after `warmup` untimed ones: CUDA events on the
        launching stream, a barrier and a device synchronisation on both sides, max over ranks.
        Returns (ms per step, kernels launched by this rank, clock record of the region)."""
        torch = self.torch
        for i in range(warmup):
            step(i)
        self.barrier()
        mark = self.monitor.begin() if self.monitor else None
        l0 = self.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        self.barrier()
        launched = self.launches() - l0
        ms = self.max_over_ranks(e0.elapsed_time(e1)) / steps
        clocks = self.monitor.end(mark) if self.monitor else None
        return ms, launched, clocks

    def steps_for(self, step, seconds, warmup=3, floor=10, cap=20000):
        """How many steps fill `seconds` (the same number on every rank)."""
        ms, _, _ = self.timed(step, 3, warmup)
        return int(min(cap, max(floor, math.ceil(seconds * 1e3 / max(ms, 1e-3)))))

    def release_memory(self):
        self.torch.cuda.synchronize()
        self.wgb.lib().wholegraph_b200_drop_cached_env_func_memory()
        self.torch.cuda.empty_cache()


def load_reference_kernels():
    """The reference's own CUDA kernels compiled from its sources (cross-check library built
    beside the oracle when the reference checkout was present), or None."""
    path = os.path.join(ROOT, "oracle", "_ref", "libwg_ref_kernels.so")
    if not os.path.exists(path):
        return None
    try:
        return ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    except OSError:
        return None


# ---- gather legs (C2, C3, C3 with distinct ids, C3 on one GPU, C4) -----------------------------
def run_gather(ctx, workload, steps, warmup, *, want_e2e, want_parity, want_cpu=False, want_scatter=False,
               want_ref=False, want_floor=False, seconds=None, comm=None, world=None, rank=None):
    """One gather configuration; returns the fields of its line as a dict (on every rank)."""
    torch, wgb, tu, args = ctx.torch, ctx.wgb, ctx.tu, ctx.args
    import numpy as np
    comm = comm if comm is not None else ctx.comm
    world = world if world is not None else ctx.world
    rank = rank if rank is not None else ctx.rank
    multi = world > 1
    MT, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphDataType
    mem_type, zipf_alpha, zipf_shift = MT.MtContinuous, None, 0.0
    n_ids = args.ids or IDS_PER_RANK
    if workload == "c2":
        rows = args.rows or 10_000_000
        tab_dtype, out_dtype, tab_wg = torch.float32, torch.float16, DT.DtFloat
    elif workload in ("c3", "c3-unique", "c3-single"):
        rows = args.rows or 100_000_000
        zipf_alpha = 1.1
        tab_dtype, out_dtype, tab_wg = torch.float16, torch.float16, DT.DtHalf
    else:
        n_ids = args.ids or 4_194_304
        rows = args.rows or 240_000_000
        # Zipf-Mandelbrot shift calibrated so that a 4,194,304-id request over 240 M rows holds
        # about 30 % duplicates, the rate the configuration states.
        zipf_alpha, zipf_shift, mem_type = 1.2, 1.4e5, MT.MtDistributed
        tab_dtype, out_dtype, tab_wg = torch.bfloat16, torch.bfloat16, DT.DtBF16
    config = gather_config(workload, world, rows, n_ids)
    es_tab = torch.empty((), dtype=tab_dtype).element_size()
    es_out = torch.empty((), dtype=out_dtype).element_size()
    first_row = equal_first_rows(rows, world)
    seed_of_owner = lambda owner: 1234 + owner

    table = wgb.create_wholegraph_tensor(wgb.make_description([rows, ROW_DIM], tab_wg), comm, mem_type,
                                         wgb.WholeGraphMemoryLocation.MlDevice)
    local_rows = wgb.C.c_size_t()
    wgb.check(wgb.lib().wholegraph_tensor_get_local_entry_count(wgb.C.byref(local_rows), table), "entry_count")
    local_rows = local_rows.value
    assert local_rows == first_row[rank + 1] - first_row[rank]
    fill_shard(torch, tu, table, local_rows, ROW_DIM, tab_dtype, seed_of_owner(rank))

    batches = []
    if workload == "c2":
        for b in range(INDEX_BATCHES):
            g = torch.Generator(device="cuda").manual_seed(1 + b)
            batches.append(torch.randint(0, rows, (n_ids,), generator=g, device="cuda", dtype=torch.int64))
    else:
        perm = torch.randperm(rows, generator=torch.Generator(device="cuda").manual_seed(7), device="cuda")
        for b in range(INDEX_BATCHES):
            if workload == "c3-unique":
                lo = ((b * world + rank) * n_ids) % max(1, rows - n_ids)
                batches.append(perm[lo:lo + n_ids].clone())
            else:
                g = torch.Generator(device="cuda").manual_seed(100 + ctx.rank + 1000 * b)
                batches.append(zipf_ids(torch, n_ids, rows, zipf_alpha, perm, g, zipf_shift))
        del perm
        torch.cuda.empty_cache()
    out = torch.empty((n_ids, ROW_DIM), dtype=out_dtype, device="cuda")
    env = ctx.env
    wraps = [tu.wrap_torch_tensor(b) for b in batches]
    wout = tu.wrap_torch_tensor(out)
    stream = tu.current_stream_int()

    def step(i):
        wgb.wholegraph_gather_op(table, wraps[i % INDEX_BATCHES], wout, env, stream)

    if args.env_sweep and workload == ctx.sweep_workload:
        # Tuning sweep: one process compares settings on the same table and index batches.  The
        # library reads its WG_* variables when a communicator is created, so each setting is
        # followed by the collective call that reads them again.
        for setting in args.env_sweep.split(";"):
            pairs = dict(kv.split("=", 1) for kv in setting.split(",") if kv)
            os.environ.update(pairs)
            wgb.check(wgb.lib().wholegraph_b200_reload_tuning(comm), "reload_tuning")
            ms, _, _ = ctx.timed(step, steps, warmup)
            if ctx.rank == 0:
                print(json.dumps({"variant": pairs, "workload": config["workload"], "n_gpus": world, "steps": steps,
                                  "ms_per_step": ms,
                                  "value": world * n_ids * ROW_DIM * es_out / (ms * 1e-3) / 1e9, "unit": "GB/s"}),
                      flush=True)
        for w in wraps + [wout]:
            wgb.destroy_wholegraph_tensor(w)
        ctx.barrier()
        wgb.destroy_wholegraph_tensor(table)
        return None

    if seconds is not None:
        steps = ctx.steps_for(step, seconds, warmup)
        warmup = 3

    # ---- device-resident timing ------------------------------------------------------------
    mark_all = ctx.monitor.begin() if ctx.monitor else None
    ms_step, launches, clocks = ctx.timed(step, steps, warmup)
    out_bytes = n_ids * ROW_DIM * es_out
    value = world * out_bytes / (ms_step * 1e-3) / 1e9
    res = {"metric": "gathered embedding GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
           "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": {"c2": "f32->f16", "c4": "bf16"}.get(workload, "f16"), "data": "synthetic", "config": config,
           "gpu_launches": int(launches)}

    # ---- parity: sampled output rows against the table rows rebuilt from the fill seeds ------
    sample_pos = expected = None
    if want_parity:
        last = (steps - 1) % INDEX_BATCHES
        ids_last = batches[last]
        g = torch.Generator(device="cuda").manual_seed(4242 + ctx.rank)
        sample_pos = torch.randint(0, n_ids, (PARITY_SAMPLE,), generator=g, device="cuda")
        hot = torch.mode(ids_last[: min(n_ids, 262_144)]).values        # the most requested id of a prefix
        sample_pos[0] = int((ids_last == hot).nonzero()[0].item())
        sample_pos[1], sample_pos[2] = 0, n_ids - 1
        sample_ids = ids_last[sample_pos]
        src_rows = regenerate_rows(torch, sample_ids, first_row, ROW_DIM, tab_dtype, seed_of_owner)
        from oracle import oracle as orc
        src_np = src_rows.cpu().numpy() if tab_dtype != torch.bfloat16 else bits(torch, src_rows).view(np.uint16)
        expected = orc.gather(src_np, np.arange(PARITY_SAMPLE, dtype=np.int64), out_dt=int(tu.TORCH_TO_WG[out_dtype]),
                              table_bf16=(tab_dtype == torch.bfloat16))
        expected = np.ascontiguousarray(expected).view(np.int16 if es_out == 2 else np.int32)
        got = bits(torch, out[sample_pos])
        bad_rows = int((got != expected).any(axis=1).sum())
        owners = torch.bucketize(sample_ids, torch.tensor(first_row[1:], device="cuda"), right=True)
        remote = int((owners != rank).sum().item())
        res["parity"] = {
            "rows_checked": int(ctx.sum_over_ranks(PARITY_SAMPLE)) if multi else PARITY_SAMPLE,
            "mismatches": int(ctx.sum_over_ranks(bad_rows)) if multi else bad_rows,
            "rows_owned_by_other_ranks": int(ctx.sum_over_ranks(remote)) if multi else remote,
            "how": f"{PARITY_SAMPLE} output positions per rank of the last timed step (first, last, the most requested "
                   "id, random others): table rows rebuilt from the owners' fill seeds without reading the table, cast "
                   "by the CPU oracle, compared bit for bit"}
        if res["parity"]["mismatches"]:
            ctx.failures.append(f"{workload}: {res['parity']['mismatches']} gathered rows differ from the table")

    # ---- end to end: pinned host ids in, pinned host rows out, copies inside the timed region
    if want_e2e:
        res["host_buffers"] = bind_to_gpu_local_cpus(torch, ctx.local_rank)
        h_idx = [b.cpu().pin_memory() for b in batches]
        h_out = torch.empty((n_ids, ROW_DIM), dtype=out_dtype).pin_memory()
        d_idx = torch.empty_like(batches[0])
        w_didx = tu.wrap_torch_tensor(d_idx)

        def e2e_step(i):
            d_idx.copy_(h_idx[i % INDEX_BATCHES], non_blocking=True)
            wgb.wholegraph_gather_op(table, w_didx, wout, env, stream)
            h_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the caller reads the rows on the host

        for i in range(min(warmup, 3)):
            e2e_step(i)
        ctx.barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            e2e_step(i)
        ctx.barrier()
        e2e_ms = ctx.max_over_ranks((time.perf_counter() - t0) * 1e3) / steps
        res["e2e"] = {"value": world * out_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                      "h2d_bytes_per_step": n_ids * 8, "d2h_bytes_per_step": out_bytes, "ms_per_step": e2e_ms}
        if want_parity:
            got = h_out[sample_pos.cpu()].contiguous().view(torch.int16 if es_out == 2 else torch.int32).numpy()
            bad = int((got != expected).any(axis=1).sum())
            bad = int(ctx.sum_over_ranks(bad)) if multi else bad
            res["parity"]["e2e_host_rows_mismatches"] = bad
            if bad:
                ctx.failures.append(f"{workload}: {bad} rows of the end-to-end host output differ from the table")
        if want_floor:
            # What bounds e2e: every rank copying its output to pinned host memory at once, nothing else.
            def copy_step(i):
                h_out.copy_(out, non_blocking=True)
            k = ctx.steps_for(copy_step, 0.5, warmup=2, floor=5)
            ms_copy, _, _ = ctx.timed(copy_step, k, 2)
            res["d2h_floor"] = {"ms_per_copy": ms_copy, "bytes_per_rank": out_bytes,
                                "per_gpu_gbs": out_bytes / (ms_copy * 1e-3) / 1e9,
                                "node_gbs": world * out_bytes / (ms_copy * 1e-3) / 1e9,
                                "e2e_step_over_floor": e2e_ms / ms_copy,
                                "how": f"{k} back-to-back cudaMemcpyAsync device-to-host copies of the {out_bytes} B "
                                       "output into the same pinned buffer on every rank at once (CUDA events, max over ranks)"}
        wgb.destroy_wholegraph_tensor(w_didx)
        del h_idx, h_out
    # the main line's clock record spans the device-timed region and the end-to-end region
    if ctx.monitor:
        wide = ctx.monitor.end(mark_all)
        res["clocks"] = wide if (clocks is None or wide["samples"] > clocks["samples"]) else clocks

    # ---- roofline of the copy kernel -------------------------------------------------------
    algorithmic = n_ids * (ROW_DIM * es_tab + ROW_DIM * es_out + 8)   # row read + row write + id read
    if multi:
        b0 = batches[0]
        owners = torch.bucketize(b0, torch.tensor(first_row[1:], device="cuda"), right=True)
        remote = b0[owners != rank]
        remote_ids, remote_unique = int(remote.numel()), int(torch.unique(remote).numel())
        wire_row = ROW_DIM * (es_out if workload == "c4" else es_tab)   # DISTRIBUTED casts at the owner
        achieved = remote_ids * wire_row / (ms_step * 1e-3) / 1e9
        distinct = remote_unique * wire_row / (ms_step * 1e-3) / 1e9
        res["roofline"] = {
            "bound": "nvlink", "achieved": achieved, "peak": NVLINK_PEER_GBS, "unit": "GB/s",
            "frac": achieved / NVLINK_PEER_GBS, "traffic": None, "remote_ids": remote_ids,
            "remote_unique_ids": remote_unique, "achieved_distinct_rows": distinct,
            "frac_distinct_rows": distinct / NVLINK_PEER_GBS, "frac_of_nominal_900": achieved / NVLINK_NOMINAL_GBS,
            "gathered_gbs_per_gpu": value / world,
            "nvlink_bound_gathered_gbs_per_gpu": NVLINK_NOMINAL_GBS * world / (world - 1),
            "note": "achieved = ids owned by other ranks x row bytes per rank per step (rank 0, batch 0), no credit for "
                    "repeated ids, over the 770 GB/s peer copy measured on this pool (of measured); repeated remote rows "
                    "are served by caches, so a skewed list can exceed 1: achieved_distinct_rows counts every remote row "
                    "once and is the traffic that must cross the link"}
    else:
        peak, how = measured_hbm_peak()
        achieved = algorithmic / (ms_step * 1e-3) / 1e9
        res["roofline"] = {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": None, "peak_source": how, "algorithmic_bytes_per_launch": algorithmic,
            "note": "frac = algorithmic bytes (row read + row written + id read per index, no credit for repeated ids) "
                    "over CUDA-event time over the measured copy bandwidth; traffic (DRAM bytes of one launch) is "
                    "captured with ncu on a smaller table and is not scaled to this one"}

    # ---- the reference's own gather kernel on the same table and index batches (N = 1) --------
    if want_ref and not multi:
        ref = load_reference_kernels()
        if ref is None:
            res["ref_gpu_kernel"] = {"unavailable": "the cross-check library with the reference's kernels was not built"}
        else:
            ptr, _ = wgb.local_view(table)
            out_ref = torch.zeros_like(out)
            dt_tab, dt_out = int(tu.TORCH_TO_WG[tab_dtype]), int(tu.TORCH_TO_WG[out_dtype])
            vp = ctypes.c_void_p

            def ref_step(i):
                rc = ref.wgref_gather(vp(ptr), dt_tab, ctypes.c_int64(rows), ctypes.c_int64(ROW_DIM),
                                      ctypes.c_int64(ROW_DIM), ctypes.c_int64(0), vp(batches[i % INDEX_BATCHES].data_ptr()),
                                      1, ctypes.c_int64(n_ids), vp(out_ref.data_ptr()), dt_out, ctypes.c_int64(ROW_DIM),
                                      ctypes.c_int64(0), vp(stream))
                assert rc == 0
            k = max(20, steps)
            ms_ref, _, ref_clocks = ctx.timed(ref_step, k, 3)
            step((k - 1) % INDEX_BATCHES)
            torch.cuda.synchronize()
            same = bool(torch.equal(out.view(torch.int16), out_ref.view(torch.int16)))
            res["ref_gpu_kernel"] = {
                "what": "gather_temp_func of the reference (cpp/src/wholegraph_tensor_ops/functions/gather_scatter_func.cuh) "
                        "compiled for sm_100a from its own sources, same table, index batches and stream",
                "ms": ms_ref, "value": out_bytes / (ms_ref * 1e-3) / 1e9, "unit": "GB/s", "launches": k,
                "ratio": ms_ref / ms_step, "output_identical": same, "clocks": ref_clocks}
            if not same:
                ctx.failures.append(f"{workload}: output differs from the reference kernel's")
            del out_ref

    # ---- CPU oracle beside it (rank 0, N = 1 only) ----------------------------------------
    if want_cpu and not multi:
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
        res["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                               "sample": f"first {sample_rows} table rows on the host, {n_ids} ids, best of {reps} passes "
                                         f"({best * 1e3:.1f} ms) of the CPU oracle's gather with cast to fp16"}

    # ---- scatter of the same configuration: unique-id fp16 rows into the fp32 table (N = 1) ----
    if want_scatter and not multi:
        res["scatter"] = run_scatter_on(ctx, table, rows, n_ids, tab_dtype, seconds or ctx.args.extra_seconds)

    for w in wraps + [wout]:
        wgb.destroy_wholegraph_tensor(w)
    ctx.barrier()
    wgb.destroy_wholegraph_tensor(table)
    del out, batches
    ctx.release_memory()
    return res


def run_scatter_on(ctx, table, rows, n_ids, tab_dtype, seconds):
    """C2 scatter: `n_ids` unique-index fp16 rows uniform(-1, 1) into the fp32 table (cast fused
    into the copy), four index / row batches cycled; parity = the scattered rows read back."""
    torch, wgb, tu = ctx.torch, ctx.wgb, ctx.tu
    import numpy as np
    in_dtype = torch.float16
    perm = torch.randperm(rows, generator=torch.Generator(device="cuda").manual_seed(11), device="cuda")
    id_batches = [perm[b * n_ids:(b + 1) * n_ids].clone() for b in range(INDEX_BATCHES)]
    del perm
    row_batches = []
    for b in range(2):
        g = torch.Generator(device="cuda").manual_seed(20 + b)
        row_batches.append(torch.empty((n_ids, ROW_DIM), dtype=torch.float32, device="cuda")
                           .uniform_(-1, 1, generator=g).to(in_dtype))
    wi = [tu.wrap_torch_tensor(b) for b in id_batches]
    wr = [tu.wrap_torch_tensor(b) for b in row_batches]
    stream = tu.current_stream_int()

    def step(i):
        wgb.wholegraph_scatter_op(wr[i % 2], wi[i % INDEX_BATCHES], table, ctx.env, stream)

    steps = ctx.steps_for(step, seconds)
    ms, launches, clocks = ctx.timed(step, steps, 3)
    # parity: what the last step wrote, read back with a gather, against the oracle's cast of the input rows
    last = steps - 1
    back = torch.empty((n_ids, ROW_DIM), dtype=tab_dtype, device="cuda")
    tu.gather(table, id_batches[last % INDEX_BATCHES], back, ctx.env)
    torch.cuda.synchronize()
    from oracle import oracle as orc
    pos = torch.randint(0, n_ids, (PARITY_SAMPLE,), generator=torch.Generator(device="cuda").manual_seed(5), device="cuda")
    rows_np = row_batches[last % 2][pos].cpu().numpy()
    want = np.zeros((PARITY_SAMPLE, ROW_DIM), dtype=np.float32)
    orc.scatter(rows_np, np.arange(PARITY_SAMPLE, dtype=np.int64), want)
    bad = int((bits(torch, back[pos]) != want.view(np.int32)).any(axis=1).sum())
    if bad:
        ctx.failures.append(f"scatter: {bad} scattered rows differ from the oracle")
    es_in, es_tab = 2, torch.empty((), dtype=tab_dtype).element_size()
    algorithmic = n_ids * (ROW_DIM * es_in + ROW_DIM * es_tab + 8)
    peak, how = measured_hbm_peak()
    achieved = algorithmic / (ms * 1e-3) / 1e9
    for w in wi + wr:
        wgb.destroy_wholegraph_tensor(w)
    return {"metric": "scattered embedding GB/s", "value": n_ids * ROW_DIM * es_in / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "ms_per_step": ms, "steps": steps, "gpu_launches": int(launches), "clocks": clocks,
            "config": {"workload": f"C2 scatter: {n_ids} unique int64 ids, fp16 rows uniform(-1,1) into the {rows} x "
                                   f"{ROW_DIM} fp32 CONTINUOUS/DEVICE table"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": how, "algorithmic_bytes_per_launch": algorithmic,
                         "note": "row read + row written + id read per index; the table rows are written in full, so no "
                                 "read of the old contents is counted"},
            "parity": {"rows_checked": PARITY_SAMPLE, "mismatches": bad,
                       "how": "rows of the last timed scatter read back through wholegraph_gather and compared bit for bit "
                              "with the CPU oracle's scatter (fp16 -> fp32) of the same input rows"}}


# ---- C5: sparse Lazy Adam ----------------------------------------------------------------------
def run_sparse_adam(ctx, steps, warmup, seconds=None, want_ref=False):
    """C5: one Lazy Adam step per bench step on a DISTRIBUTED fp32 table of dim 256; every rank
    feeds 2,097,152 fp32 gradient rows at Zipf(1.1) ids; duplicates are summed before the update.
    Parity: one step on a sample of ids (the hottest one included) against the CPU oracle applied
    to the rows as they were before the step."""
    torch, dist, wgb, tu, args = ctx.torch, ctx.dist, ctx.wgb, ctx.tu, ctx.args
    import ctypes as C
    import numpy as np
    world, rank, multi, comm = ctx.world, ctx.rank, ctx.multi, ctx.comm
    dim = 256
    rows = args.rows or (50_000_000 if world == 8 else 6_250_000 * world)   # 6.25 M rows per GPU
    n = args.ids or 2_097_152
    lr = 1e-3
    DT, MT, ML = wgb.WholeGraphDataType, wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation
    env = ctx.env
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
    distinct_rank0 = int(torch.unique(batches[0][0]).numel())
    stream = tu.current_stream_int()

    def step(i):
        _, _, wi, wg = batches[i % 2]
        wgb.EmbeddingGatherGradientApply(emb, wi, wg, False, lr, env, stream)

    state_t = {nm: wgb.embedding_state(emb, nm) for nm in ("m", "v")}
    beta_t = wgb.embedding_state(emb, "beta12t")

    # ---- parity of one step on sampled ids ---------------------------------------------------
    parity = None
    if not args.no_parity:
        from oracle import oracle as orc
        ids0, grads0 = batches[0][0], batches[0][1]
        raw = torch.empty(1024, dtype=torch.int64, device="cuda")
        if rank == 0:
            pick = torch.randint(0, n, (1024,), generator=torch.Generator(device="cuda").manual_seed(99), device="cuda")
            raw.copy_(ids0[pick])
            raw[0] = torch.mode(ids0[:262_144]).values        # the most frequent id: a run far longer than a block
        if multi:
            dist.broadcast(raw, 0)
        sample = torch.unique(raw)                              # ascending, identical on every rank
        k = int(sample.numel())

        def read_rows():
            got = {}
            for nm, t, width in [("w", table, dim), ("m", state_t["m"], dim), ("v", state_t["v"], dim), ("beta", beta_t, 2)]:
                buf = torch.empty((k, width), dtype=torch.float32, device="cuda")
                tu.gather(t, sample, buf, env)
                torch.cuda.synchronize()
                got[nm] = buf.cpu().numpy()
            return got

        before = read_rows()
        mine = torch.isin(ids0, sample)
        ids_s, grads_s = ids0[mine].cpu().numpy(), grads0[mine].cpu().numpy()
        longest = int(ctx.max_over_ranks(float(np.unique(ids_s, return_counts=True)[1].max()) if len(ids_s) else 0.0))
        presum = os.environ.get("WG_GRADIENT_PRESUM", "1") != "0" and multi
        if multi:
            if presum:   # this rank's duplicates first, in arrival order (runs over 256 rows block by block)
                u, sums = orc.dedup_gradients(ids_s, grads_s, block=256) if len(ids_s) else (ids_s, grads_s)
                present = torch.zeros(k, dtype=torch.int64, device="cuda")
                dense = torch.zeros((k, dim), dtype=torch.float32, device="cuda")
                if len(u):
                    slot = torch.searchsorted(sample, torch.from_numpy(u).cuda())
                    present[slot] = 1
                    dense[slot] = torch.from_numpy(sums).cuda()
                all_present = [torch.zeros_like(present) for _ in range(world)]
                all_dense = [torch.zeros_like(dense) for _ in range(world)]
                dist.all_gather(all_present, present)
                dist.all_gather(all_dense, dense)
                cat_ids = np.concatenate([sample[p.bool()].cpu().numpy() for p in all_present])
                cat_rows = np.concatenate([d[p.bool()].cpu().numpy() for p, d in zip(all_present, all_dense)])
            else:        # every row routed: one chain in rank-then-arrival order
                counts = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(world)]
                dist.all_gather(counts, torch.tensor([len(ids_s)], dtype=torch.int64, device="cuda"))
                cap = int(max(c.item() for c in counts))
                pid = torch.full((cap,), -1, dtype=torch.int64, device="cuda")
                pgr = torch.zeros((cap, dim), dtype=torch.float32, device="cuda")
                pid[:len(ids_s)] = torch.from_numpy(ids_s).cuda()
                pgr[:len(ids_s)] = torch.from_numpy(grads_s).cuda()
                all_id = [torch.zeros_like(pid) for _ in range(world)]
                all_gr = [torch.zeros_like(pgr) for _ in range(world)]
                dist.all_gather(all_id, pid)
                dist.all_gather(all_gr, pgr)
                cat_ids = np.concatenate([a[:int(c.item())].cpu().numpy() for a, c in zip(all_id, counts)])
                cat_rows = np.concatenate([a[:int(c.item())].cpu().numpy() for a, c in zip(all_gr, counts)])
        else:
            cat_ids, cat_rows = ids_s, grads_s
        uniq, sums = orc.dedup_gradients(cat_ids, cat_rows, block=256)
        step(0)
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
        after = read_rows()
        sample_np = sample.cpu().numpy()
        w = before["w"].copy()
        state = np.concatenate([before["m"], before["v"]], axis=1)
        beta = before["beta"].copy()
        orc.optimizer_apply(2, np.searchsorted(sample_np, uniq).astype(np.int64), sums, w, lr=lr, state=state, v_offset=dim,
                            beta12t=beta)
        bad, worst = 0, 0.0
        for nm, want in [("w", w), ("m", state[:, :dim]), ("v", state[:, dim:]), ("beta", beta)]:
            got = after[nm]
            diff = got.view(np.int32) != np.ascontiguousarray(want).view(np.int32)
            bad += int(diff.sum())
            denom = np.maximum(np.abs(want), 1e-7)
            worst = max(worst, float((np.abs(got - want) / denom).max()))
        touched = int(len(uniq))
        parity = {"rows_checked": touched, "elements_checked": touched * (3 * dim + 2), "mismatches": bad,
                  "max_relative_error": worst, "tolerance": 1e-6,
                  "longest_run_checked": longest,
                  "how": "one step on a sample of ids (the most frequent id included): weights, m, v and the beta powers "
                         "read through wholegraph_gather before and after; the CPU oracle sums the sampled ids' gradient rows "
                         + ("per rank in arrival order, then the per-rank sums in rank order, " if presum else
                            "in rank-then-arrival order, ") +
                         "runs longer than 256 rows block by block, and applies Lazy Adam; compared bit for bit"}
        if worst > 1e-6:
            ctx.failures.append(f"c5: optimizer result off by {worst:.3g} relative")

    if seconds is not None:
        steps = ctx.steps_for(step, seconds, warmup)
        warmup = 3
    ms_step, launches, clocks = ctx.timed(step, steps, warmup)
    peak, how = measured_hbm_peak()
    # per rank: every raw gradient row read once (1024 B) + 7184 B per distinct row updated; with
    # several ranks the distinct rows of rank 0's batch stand for the rows one owner updates
    algorithmic = n * dim * 4 + distinct_rank0 * 7184
    achieved = algorithmic / (ms_step * 1e-3) / 1e9
    res = {"metric": "sparse-Adam rows/s", "value": world * n / (ms_step * 1e-3), "unit": "rows/s",
           "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": f"C5: Lazy Adam on a {rows} x {dim} fp32 DISTRIBUTED table over {world} GPUs, "
                                  f"{n} gradient rows N(0,1e-3) per rank per step at Zipf(1.1) ids, lr 1e-3",
                      "distinct_ids_rank0_batch0": distinct_rank0},
           "gpu_launches": int(launches), "clocks": clocks,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "traffic": None, "peak_source": how, "algorithmic_bytes_per_launch": algorithmic,
                        "note": "per rank per step: 1024 B per raw gradient row + 7184 B per distinct updated row "
                                "(distinct ids of rank 0's first batch)"}}
    if parity is not None:
        res["parity"] = parity

    # ---- the reference's own dedup + optimizer kernels on the same gradients (N = 1) ----------
    if want_ref and not multi:
        ref = load_reference_kernels()
        if ref is None:
            res["ref_gpu_kernel"] = {"unavailable": "the cross-check library with the reference's kernels was not built"}
        else:
            w_ptr, _ = wgb.local_view(table)
            state_root = C.c_void_p(wgb.lib().wholegraph_tensor_get_root(state_t["m"]))
            s_ptr, _ = wgb.local_view(state_root)
            beta_root = C.c_void_p(wgb.lib().wholegraph_tensor_get_root(beta_t))
            b_ptr, _ = wgb.local_view(beta_root)
            dedup_ids = torch.empty(n, dtype=torch.int64, device="cuda")
            dedup_grads = torch.empty((n, dim), dtype=torch.float32, device="cuda")
            vp, i64 = ctypes.c_void_p, ctypes.c_int64
            ref.wgref_dedup_gradients.restype = ctypes.c_long

            def ref_step(i):
                ids, grads, _, _ = batches[i % 2]
                u = ref.wgref_dedup_gradients(vp(ids.data_ptr()), i64(n), vp(grads.data_ptr()), i64(dim), i64(dim),
                                              vp(dedup_ids.data_ptr()), vp(dedup_grads.data_ptr()),
                                              ctypes.cast(env, vp), vp(stream))
                assert u > 0
                rc = ref.wgref_optimizer_step(2, vp(dedup_ids.data_ptr()), vp(dedup_grads.data_ptr()), i64(u), vp(w_ptr), 1,
                                              vp(s_ptr), vp(b_ptr), i64(0), dim, dim, dim, ctypes.c_float(lr),
                                              ctypes.c_float(0.0), ctypes.c_float(1e-8), ctypes.c_float(0.9),
                                              ctypes.c_float(0.999), ctypes.c_float(0.99), 0, vp(stream))
                assert rc == 0
            ms_ref, _, ref_clocks = ctx.timed(ref_step, 5, 2)
            res["ref_gpu_kernel"] = {
                "what": "the reference's dedup_indice_and_gradients (radix sort, unique, one block per distinct id adding its "
                        "rows one after the other) followed by its lazy_adam_optimizer_step_kernel, compiled for sm_100a from "
                        "its own sources, same gradients, same table and state memory",
                "ms": ms_ref, "value": n / (ms_ref * 1e-3), "unit": "rows/s", "launches": 5, "ratio": ms_ref / ms_step,
                "clocks": ref_clocks}
            del dedup_ids, dedup_grads

    for _, _, wi, wg in batches:
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wg)
    ctx.barrier()
    wgb.destroy_embedding(emb)
    wgb.lib().wholegraph_destroy_embedding_optimizer(opt)
    del batches
    ctx.release_memory()
    return res


def run_cached_gather(ctx, steps, warmup):
    """Cached embedding gather on one GPU: a 10 M x 128 fp32 table behind a set-associative cache
    holding one row in eight (sets of 32 lines over 256 rows), 1,048,576 Zipf(1.1) ids per step
    over a seeded permutation, fp32 output.  Timed twice: lookups only (adjust_cache = False, after
    the cache has been warmed) and with the LFU update of every step inside the timed region."""
    torch, wgb, tu, args, comm = ctx.torch, ctx.wgb, ctx.tu, ctx.args, ctx.comm
    import ctypes as C
    dim = ROW_DIM
    rows = args.rows or 10_000_000
    n = args.ids or IDS_PER_RANK
    DT, MT, ML, AT = (wgb.WholeGraphDataType, wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation,
                      wgb.WholeGraphAccessType)
    env = ctx.env
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

    def lookup_step(i):
        wgb.EmbeddingGatherForward(emb, wraps[i % INDEX_BATCHES], wout, False, env, stream)

    def adjust_step(i):
        wgb.EmbeddingGatherForward(emb, wraps[i % INDEX_BATCHES], wout, True, env, stream)

    for i in range(2 * INDEX_BATCHES):      # warm the cache with every batch
        adjust_step(i)
    mark = ctx.monitor.begin()
    ms_lookup, launches, _ = ctx.timed(lookup_step, steps, warmup)
    ms_adjust, _, _ = ctx.timed(adjust_step, steps, warmup)
    clocks = ctx.monitor.end(mark)
    tags = wgb.embedding_cache_tensors(emb)[0]
    sets = wgb.lib().wholegraph_tensor_get_tensor_description(tags).contents.sizes[0]
    peak, how = measured_hbm_peak()
    algorithmic = n * (2 * dim * 4 + 8 + 64)       # row read + row write + id + one 64-byte tag set per id
    achieved = algorithmic / (ms_lookup * 1e-3) / 1e9
    line = {"metric": "gathered embedding GB/s", "value": n * dim * 4 / (ms_lookup * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms_lookup,
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
    for w in wraps:
        wgb.destroy_wholegraph_tensor(w)
    wgb.destroy_wholegraph_tensor(wout)
    wgb.destroy_embedding(emb)
    wgb.destroy_cache_policy(policy)
    return line


def run_append_unique(ctx, steps, warmup):
    """graph_append_unique on one GPU with the shapes of the last hop of a [15, 10, 5] fan-out from 1,024
    seeds: 153,600 distinct int64 target nodes and 768,000 sampled neighbours (Zipf(1.2) over 240 M node ids,
    some of them targets).  A step is one call, output allocation and its host synchronisations included."""
    torch, wgb, tu, args = ctx.torch, ctx.wgb, ctx.tu, ctx.args
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
    env, stream = ctx.env, tu.current_stream_int()
    slot = wgb.OutputSlot()
    seen = {}

    def step(i):
        wgb.append_unique(wt, wn[i % INDEX_BATCHES], slot, wm, env, stream)
        seen["n"] = slot.description.sizes[0]
        wgb.release_output(slot)

    ms, launches, clocks = ctx.timed(step, steps, warmup)
    n_unique = seen["n"]
    peak, how = measured_hbm_peak()
    m = t_count + n_count
    algorithmic = m * 8 + n_count * 4 + n_unique * 8      # ids read once, mapping and list written once
    achieved = algorithmic / (ms * 1e-3) / 1e9
    line = {
        "metric": "append-unique nodes/s", "value": m / (ms * 1e-3), "unit": "nodes/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": {"workload": f"graph_append_unique: {t_count} distinct int64 targets + {n_count} neighbours "
                               f"(Zipf(1.2, shift 1.4e5) over {nodes} node ids, 1/8 of them targets), with mapping",
                   "unique_nodes_last_step": int(n_unique)},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": how, "algorithmic_bytes_per_launch": algorithmic,
                     "note": "ids read once, mapping and node list written once; the radix sort's passes and the "
                             "host synchronisations are overhead, so this op is latency-bound at this size"}}
    for w in [wt, wm] + wn:
        wgb.destroy_wholegraph_tensor(w)
    return line


def run_peer_copy(ctx, steps, warmup):
    """The NVLink denominator: every rank copies 1 GiB of its right-hand neighbour's shard of a
    CONTINUOUS/DEVICE allocation (one mapped range, peer pages behind it) into local memory with a
    plain asynchronous memcpy, all ranks at once; GB/s per direction per GPU."""
    torch, wgb = ctx.torch, ctx.wgb
    import ctypes as C
    world, rank = ctx.world, ctx.rank
    per_rank = 1 << 30
    desc = wgb.make_description([world * (per_rank // 256), 256], wgb.WholeGraphDataType.DtInt8)
    table = wgb.create_wholegraph_tensor(desc, ctx.comm, wgb.WholeGraphMemoryType.MtContinuous,
                                         wgb.WholeGraphMemoryLocation.MlDevice)
    handle = C.c_void_p(wgb.lib().wholegraph_tensor_get_memory_handle(table))
    base = C.c_void_p()
    wgb.check(wgb.lib().wholegraph_get_global_pointer(C.byref(base), handle), "global_pointer")
    local = torch.empty(per_rank, dtype=torch.uint8, device="cuda")
    peer = (rank + 1) % world
    src = base.value + peer * per_rank
    stream = C.c_void_p(ctx.tu.current_stream_int())

    def step(i):
        wgb.check(wgb.lib().wholegraph_b200_memcpy_async(C.c_void_p(local.data_ptr()), C.c_void_p(src), per_rank, stream),
                  "memcpy_async")

    ms, _, clocks = ctx.timed(step, steps, warmup)
    gbs = per_rank / (ms * 1e-3) / 1e9
    line = {"metric": "peer copy GB/s per direction per GPU", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"peer copy: every one of {world} ranks reads 1 GiB of its neighbour's shard of a "
                                   f"CONTINUOUS/DEVICE allocation into local memory (cudaMemcpyAsync), all at once; "
                                   f"time = max over ranks"},
            "gpu_launches": 0, "clocks": clocks,
            "roofline": {"bound": "nvlink", "achieved": gbs, "peak": NVLINK_NOMINAL_GBS, "unit": "GB/s",
                         "frac": gbs / NVLINK_NOMINAL_GBS, "traffic": None,
                         "note": "against the nominal 900 GB/s per direction per GPU"}}
    ctx.barrier()
    wgb.destroy_wholegraph_tensor(table)
    return line


def compact(res, keys=("metric", "value", "unit", "ms_per_step", "steps", "gpu_launches", "clocks", "roofline", "parity",
                       "config", "ref_gpu_kernel", "d2h_floor")):
    """The fields of a configuration's line that go into `extra`."""
    return {k: res[k] for k in keys if k in res}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

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

    if multi:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        raw = wgb.unique_id_to_bytes(wgb.create_unique_id()) if rank == 0 else bytes(128)
        buf = torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()
        dist.broadcast(buf, 0)
        uid = wgb.unique_id_from_bytes(buf.cpu().numpy().tobytes())
        comm = wgb.create_communicator(uid, rank, world)
    else:
        comm = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    ctx = Context(args, torch, dist, wgb, tu, comm, world, rank, local_rank)
    ctx.sweep_workload = workload

    line = None
    if workload == "p2p":
        if not multi:
            raise SystemExit("the p2p workload needs more than one GPU")
        line = run_peer_copy(ctx, args.steps, args.warmup)
    elif workload in ("cache", "unique"):
        if multi:
            raise SystemExit(f"the {workload} workload runs on one GPU")
        line = run_cached_gather(ctx, args.steps, args.warmup) if workload == "cache" else \
            run_append_unique(ctx, args.steps, args.warmup)
    elif workload == "c5":
        line = run_sparse_adam(ctx, args.steps, args.warmup, want_ref=not args.no_extras)
    elif workload in ("c2", "c3", "c3-unique", "c4"):
        auto = args.workload == "auto"
        one_rank_exchange = os.environ.get("WG_SINGLE_RANK_EXCHANGE") == "1" and workload == "c4"
        if workload != "c2" and not multi and not one_rank_exchange:
            raise SystemExit(f"the {workload} workload needs more than one GPU (c4 also runs on one GPU with "
                             "WG_SINGLE_RANK_EXCHANGE=1: the exchange code with the rank as its own peer, for profiling)")
        line = run_gather(ctx, workload, args.steps, args.warmup, want_e2e=not args.no_e2e,
                          want_parity=not args.no_parity, want_cpu=not args.no_cpu_baseline,
                          want_scatter=auto and not args.no_extras, want_ref=not args.no_extras,
                          want_floor=multi and not args.no_extras)
        if line is not None and auto and not args.no_extras:
            extra = {}
            if "scatter" in line:
                extra["scatter"] = line.pop("scatter")
            if "ref_gpu_kernel" in line:
                extra["ref_gpu_kernel_gather"] = line.pop("ref_gpu_kernel")
            if "d2h_floor" in line:
                extra["d2h_floor"] = line.pop("d2h_floor")
            sec = args.extra_seconds

            def leg(name, fn):
                try:
                    got = fn()
                    if got is not None:
                        extra[name] = compact(got)
                except Exception as exc:   # an extra never takes the main line down, but it fails the run
                    extra[name] = {"error": f"{type(exc).__name__}: {exc}"}
                    ctx.failures.append(f"{name}: {type(exc).__name__}: {exc}")
                    try:
                        ctx.release_memory()
                    except Exception:
                        pass
            if multi:
                leg("c3_unique", lambda: run_gather(ctx, "c3-unique", 0, 3, want_e2e=False,
                                                    want_parity=not args.no_parity, seconds=sec))
                solo = wgb.create_communicator(wgb.UniqueId(), 0, 1)
                leg("c3_single_gpu", lambda: run_gather(ctx, "c3-single", 0, 3, want_e2e=False, want_parity=False,
                                                        seconds=sec, comm=solo, world=1, rank=0))
                wgb.destroy_communicator(solo)
                if "c3_single_gpu" in extra and "value" in extra["c3_single_gpu"]:
                    line["config"]["c3_single_gpu_gbs"] = ctx.min_over_ranks(extra["c3_single_gpu"]["value"])
                leg("c4", lambda: run_gather(ctx, "c4", 0, 3, want_e2e=False, want_parity=not args.no_parity,
                                             seconds=sec))
            leg("c5", lambda: run_sparse_adam(ctx, 0, 3, seconds=sec, want_ref=True))
            line["extra"] = extra
    if line is not None and rank == 0:
        if ctx.failures:
            line["failures"] = ctx.failures
        print(json.dumps(line), flush=True)
    if ctx.monitor:
        ctx.monitor.close()
    ctx.barrier()
    wgb.destroy_communicator(comm)
    if multi:
        dist.destroy_process_group()
    if ctx.failures:
        sys.stderr.write("bench.py: " + "; ".join(ctx.failures) + "\n")
        raise SystemExit(1)


if __name__ == "__main__":
    main()
