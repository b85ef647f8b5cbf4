"""Multi-GPU parity: CONTINUOUS (direct NVLink loads through one mapped range), CHUNKED (one
base pointer per rank) and DISTRIBUTED (NCCL exchange) gather / scatter against the CPU oracle.
One process per GPU, as the reference's tests do with fork (cpp/src/parallel_utils.cpp:35-89).
Skipped on boxes with a single GPU."""
import os
import subprocess
import sys
import tempfile
import time

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _device_count():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


# A suffix after the last dash selects a tuning switch of the library for that scenario (the
# worker sets the variable and has the library read it again): -keepdups routes duplicates as
# the reference does, -hostcounts exchanges the counts of a distributed gather through the host,
# -nccl moves rows by NCCL instead of peer stores, -nopresum routes every gradient row (one
# summation chain per id), -peerpush writes gradient sums straight into the owner's arena region.
SCENARIOS = ["continuous", "distributed", "distributed-keepdups", "distributed-hostcounts", "distributed-nccl", "distributed-registers", "unequal-registers", "chunked",
             "optimizer", "optimizer-nopresum", "optimizer-peerpush", "cache", "fileio", "unequal", "unequal-nccl",
             "unequal-keepdups", "roundrobin", "hosttable", "nodecache", "stated-size"]


@pytest.mark.parametrize("scenario", SCENARIOS + ["all-in-one"])
def test_multi_gpu_gather_scatter(scenario):
    """One process per GPU.  `all-in-one` runs every scenario in ONE set of processes (one library
    load and one communicator for all of them): select it with WG_TEST_ALL_IN_ONE=1, which skips
    the separate runs; without the variable it is skipped."""
    world = min(_device_count(), int(os.environ.get("WG_TEST_WORLD", "8")))
    if world < 2:
        pytest.skip("needs at least two GPUs")
    together = os.environ.get("WG_TEST_ALL_IN_ONE") == "1"
    if (scenario == "all-in-one") != together:
        pytest.skip("runs with WG_TEST_ALL_IN_ONE=1" if scenario == "all-in-one" else "covered by all-in-one")
    if scenario == "all-in-one":
        scenario = ",".join(SCENARIOS)
    with tempfile.TemporaryDirectory() as rdv:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        logs = [open(os.path.join(rdv, f"rank{r}.log"), "w+") for r in range(world)]
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "mg_worker.py"), str(r), str(world), rdv, scenario],
                                  env=env, stdout=logs[r], stderr=subprocess.STDOUT, text=True)
                 for r in range(world)]
        # A rank that dies leaves its peers waiting in a collective: watch all of them and
        # stop the others as soon as one fails or the time limit passes.
        deadline = time.time() + float(os.environ.get("WG_TEST_TIMEOUT", "150")) * (1 + scenario.count(","))
        while True:
            codes = [p.poll() for p in procs]
            if all(c is not None for c in codes):
                break
            if any(c not in (None, 0) for c in codes) or time.time() > deadline:
                time.sleep(2.0)
                for p in procs:
                    if p.poll() is None:
                        p.kill()
                break
            time.sleep(0.2)
        outs = []
        for p, f in zip(procs, logs):
            p.wait()
            f.seek(0)
            outs.append(f.read())
            f.close()
        keep = os.environ.get("WG_TEST_KEEP_LOGS")
        if keep:
            os.makedirs(keep, exist_ok=True)
            for r, out in enumerate(outs):
                with open(os.path.join(keep, f"mg_{'all' if ',' in scenario else scenario}_rank{r}.log"), "w") as f:
                    f.write(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0, f"rank {r} failed (exit {p.returncode}):\n{out[-3000:]}"
            assert f"rank {r} ok" in out
