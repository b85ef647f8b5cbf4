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


@pytest.mark.parametrize("scenario", ["continuous", "distributed", "distributed-keepdups", "chunked", "optimizer", "optimizer-nopresum", "optimizer-peerpush", "cache", "fileio"])
def test_multi_gpu_gather_scatter(scenario):
    world = min(_device_count(), int(os.environ.get("WG_TEST_WORLD", "8")))
    if world < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as rdv:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        if scenario.endswith("-keepdups"):       # the path that routes duplicates, as the reference does
            env["WG_GATHER_DEDUP"] = "0"
            scenario = scenario.split("-")[0]
        if scenario.endswith("-nopresum"):       # every gradient row routed, one summation chain per id
            env["WG_GRADIENT_PRESUM"] = "0"
            scenario = scenario.split("-")[0]
        if scenario.endswith("-peerpush"):       # gradient sums written straight into the owner's arena region
            env["WG_PEER_GRADIENT"] = "1"
            scenario = scenario.split("-")[0]
        logs = [open(os.path.join(rdv, f"rank{r}.log"), "w+") for r in range(world)]
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "mg_worker.py"), str(r), str(world), rdv, scenario],
                                  env=env, stdout=logs[r], stderr=subprocess.STDOUT, text=True)
                 for r in range(world)]
        # A rank that dies leaves its peers waiting in a collective: watch all of them and
        # stop the others as soon as one fails or the time limit passes.
        deadline = time.time() + float(os.environ.get("WG_TEST_TIMEOUT", "150"))
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
                with open(os.path.join(keep, f"mg_{scenario}_rank{r}.log"), "w") as f:
                    f.write(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0, f"rank {r} failed (exit {p.returncode}):\n{out[-3000:]}"
            assert f"rank {r} ok" in out
