"""Generates tests/golden/golden_small.npz: small seeded inputs and the outputs the pinned CPU
oracle gives for them.  The reference itself cannot run where this repository is authored (no GPU,
and its Python packages are not installable offline), so these vectors freeze the oracle after
it was pinned by tests/test_oracle_pins.py; the GPU tests must reproduce them bit for bit.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as orc  # noqa: E402


def cases():
    out = {}
    rng = np.random.default_rng(20240607)
    # gather with casts, negative ids included
    rows, dim, n = 512, 24, 300
    table = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    idx = rng.integers(0, rows, size=n).astype(np.int64)
    idx[::29] = -1
    out["gather_table_f32"], out["gather_idx"] = table, idx
    out["gather_out_f16"] = orc.gather(table, idx, out_dt=orc.DT_HALF)
    out["gather_out_bf16"] = orc.gather(table, idx, out_dt=orc.DT_BF16)
    out["gather_out_f64"] = orc.gather(table, idx, out_dt=orc.DT_DOUBLE)
    # scatter fp16 rows into the fp32 table at unique ids
    sidx = rng.permutation(rows)[:100].astype(np.int64)
    srows = rng.uniform(-1, 1, size=(100, dim)).astype(np.float16)
    out["scatter_idx"], out["scatter_rows_f16"] = sidx, srows
    out["scatter_table_after"] = orc.scatter(srows, sidx, table.copy())
    # integer tables
    itab = rng.integers(-2 ** 40, 2 ** 40, size=(64, 5), dtype=np.int64)
    iidx = rng.integers(0, 64, size=50).astype(np.int32)
    out["int_table"], out["int_idx"] = itab, iidx
    out["int_out_i8"] = orc.gather(itab, iidx, out_dt=orc.DT_INT8)
    out["int_out_i32"] = orc.gather(itab, iidx, out_dt=orc.DT_INT)
    # three Lazy Adam steps with duplicate ids
    rows, dim, n = 64, 12, 200
    w = rng.normal(0, 0.01, size=(rows, dim)).astype(np.float32)
    out["adam_w0"] = w.copy()
    state, beta = np.zeros((rows, 2 * dim), np.float32), np.ones((rows, 2), np.float32)
    for step in range(3):
        ids = rng.integers(0, rows, size=n).astype(np.int64)
        grads = rng.normal(0, 1e-3, size=(n, dim)).astype(np.float32)
        out[f"adam_ids_{step}"], out[f"adam_grads_{step}"] = ids, grads
        uniq, sums = orc.dedup_gradients(ids, grads)
        orc.optimizer_apply(orc.OPT_LAZY_ADAM, uniq, sums, w, lr=1e-3, state=state, v_offset=dim, beta12t=beta)
    out["adam_w3"], out["adam_state3"], out["adam_beta3"] = w, state, beta
    return out


if __name__ == "__main__":
    path = os.path.join(HERE, "golden_small.npz")
    np.savez_compressed(path, **cases())
    print(path, os.path.getsize(path), "bytes")
