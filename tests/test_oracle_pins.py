"""Pins the CPU oracle against the reference's own known-answer constructions (no GPU).

The reference's tests do not hold golden byte vectors: they fill tables with closed-form values
and compare bitwise against the same closed form (cpp/tests/wholegraph_tensor_ops/
embedding_test_utils.cu:186-247, :390-420; python/wholegraph-torch/tests/wholegraph_torch/ops/
test_wholegraph_gather_scatter.py:36-140), and check the optimizers against a CPU optimizer
(wholegraph_embedding_gradient_apply_tests.cu:170-380, :448-488).  Those constructions are
re-derived here in plain numpy, independently of the oracle's C code, and the oracle has to
reproduce them bit for bit."""
import numpy as np
import pytest
import torch

MANTISSA = {1: 23, 2: 10, 3: 52, 4: 7}  # float, half, double, bf16


def to_dtype_bits(values_f64, dt):
    """Cast exact float64 values to wholegraph dtype `dt` the way CUDA's static_cast does."""
    if dt == 1:
        return values_f64.astype(np.float32)
    if dt == 3:
        return values_f64.astype(np.float64)
    f32 = values_f64.astype(np.float32)
    t = torch.from_numpy(f32)
    if dt == 2:
        return t.to(torch.float16).numpy()
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def reference_generator_table(rows, dim, dt):
    """Element (r, c) = cast(r & ((1 << (M + 1)) - 1)) for float types, cast(r) for integers
    (embedding_test_utils.cu:186-227: the last assignment overrides the hash with the row id)."""
    r = np.arange(rows, dtype=np.int64)
    if dt in MANTISSA:
        vals = (r & ((1 << (MANTISSA[dt] + 1)) - 1)).astype(np.float64)
        col = to_dtype_bits(vals, dt)
    else:
        col = r.astype({5: np.int32, 6: np.int64, 7: np.int16, 8: np.int8}[dt])
    return np.repeat(col[:, None], dim, axis=1).copy()


def expected_after_cast(table_col_values, src_dt, dst_dt):
    """What the reference expects in the output: generate in the table dtype, cast to the output
    dtype through fp32 when a 16-bit float is involved (device_matrix_type_cast)."""
    if src_dt in MANTISSA:
        if src_dt == 1:
            wide = table_col_values.astype(np.float64)
        elif src_dt == 3:
            wide = table_col_values
        elif src_dt == 2:
            wide = table_col_values.astype(np.float64)
        else:
            wide = (table_col_values.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        if dst_dt in (2, 4) and src_dt == 3:
            wide = wide.astype(np.float32).astype(np.float64)  # double -> float -> half: two roundings
        return to_dtype_bits(wide, dst_dt)
    return table_col_values.astype({5: np.int32, 6: np.int64, 7: np.int16, 8: np.int8}[dst_dt])


@pytest.mark.parametrize("dim,stride,offset", [(1, 1, 0), (11, 11, 0), (32, 32, 0), (127, 127, 0), (128, 128, 0),
                                               (129, 129, 0), (513, 513, 0), (32, 33, 0), (11, 12, 0), (64, 80, 16)])
@pytest.mark.parametrize("src_dt,dst_dt", [(1, 1), (2, 2), (1, 2), (2, 1), (4, 4), (4, 1), (1, 4), (3, 2), (3, 1),
                                           (2, 4), (5, 5), (6, 6), (8, 6), (6, 8), (7, 5)])
def test_gather_reproduces_the_reference_generator(orc, dim, stride, offset, src_dt, dst_dt):
    rows, n = 70_001, 4_097          # more rows than any 16-bit mantissa holds, so the mask matters
    rng = np.random.default_rng(dim + 10 * src_dt + 100 * dst_dt)
    table = reference_generator_table(rows, dim, src_dt)
    storage = np.zeros(offset + rows * stride, dtype=table.dtype)
    view = storage[offset:offset + rows * stride].reshape(rows, stride)[:, :dim]
    view[:] = table
    idx = rng.integers(0, rows, size=n).astype(np.int64 if dim % 2 else np.int32)
    got = orc.gather(view, idx, out_dt=dst_dt, table_bf16=(src_dt == 4))
    with np.errstate(over="ignore"):
        want_col = expected_after_cast(table[idx, 0], src_dt, dst_dt)
    assert got.shape == (n, dim)
    assert np.array_equal(got.view(want_col.dtype), np.repeat(want_col[:, None], dim, axis=1))


def test_scatter_then_gather_reproduces_the_generator(orc):
    """Reference scatter test: scatter generator rows (duplicates are benign because the value
    depends only on the index), gather them back, compare bitwise
    (wholegraph_scatter_tests.cu:125-279)."""
    rows, dim, n = 30_000, 129, 9_999
    rng = np.random.default_rng(3)
    idx = rng.integers(0, rows, size=n).astype(np.int64)
    src = reference_generator_table(rows, dim, 1)[idx]           # row value = its index
    table = np.zeros((rows, dim), dtype=np.float16)
    orc.scatter(src, idx, table)
    back = orc.gather(table, idx, out_dt=1)
    with np.errstate(over="ignore"):
        want = src.astype(np.float16).astype(np.float32)
    assert np.array_equal(back, want)


def test_python_reference_construction_index_plus_column(orc):
    """value(row, col) = row + col in fp32; gather equals torch-CPU indexing
    (test_wholegraph_gather_scatter.py:36-140)."""
    rows, dim = 50_000, 64
    table = (np.arange(rows, dtype=np.float32)[:, None] + np.arange(dim, dtype=np.float32)[None, :])
    idx = np.random.default_rng(1).integers(0, rows, size=8_192)
    got = orc.gather(table, idx)
    assert np.array_equal(got, torch.from_numpy(table)[torch.from_numpy(idx)].numpy())
    out = np.full((3, dim), -1, dtype=np.float32)
    orc.gather(table, np.array([5, -1, 7]), out=out)             # negative index: row untouched
    assert np.array_equal(out[1], np.full(dim, -1, dtype=np.float32)) and out[0, 0] == 5 and out[2, 3] == 10


def test_float_conversions_cover_every_exponent_class(orc):
    bits = np.concatenate([np.arange(0, 2 ** 32, 40_009, dtype=np.uint64),
                           np.array([0x33000000, 0x33000001, 0x387FE000, 0x387FF000, 0x477FE000, 0x477FF000,
                                     0x47800000, 0x7F800000, 0xFF800000, 0x00000001, 0x80000000], dtype=np.uint64)])
    x = bits.astype(np.uint32).view(np.float32)
    x = x[~np.isnan(x)]
    with np.errstate(over="ignore"):
        want_h = x.astype(np.float16).view(np.uint16)
    got_h = orc.gather(x.reshape(-1, 1), np.arange(x.size), out_dt=2).view(np.uint16).ravel()
    assert np.array_equal(got_h, want_h)
    want_b = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got_b = orc.gather(x.reshape(-1, 1), np.arange(x.size), out_dt=4).ravel()
    assert np.array_equal(got_b, want_b)
    # widening back is exact
    h = np.arange(0, 2 ** 16, dtype=np.uint16).view(np.float16)
    h = h[~np.isnan(h)]
    assert np.array_equal(orc.gather(h.reshape(-1, 1), np.arange(h.size), out_dt=1).ravel(), h.astype(np.float32))
    # NaN maps to the canonical 0x7FFF as the device conversion does
    nan = np.array([[np.nan]], dtype=np.float32)
    assert orc.gather(nan, np.array([0]), out_dt=2).view(np.uint16)[0, 0] == 0x7FFF
    assert orc.gather(nan, np.array([0]), out_dt=4)[0, 0] == 0x7FFF


def test_mixing_float_and_integer_is_rejected(orc):
    with pytest.raises(TypeError):
        orc.gather(np.zeros((4, 4), dtype=np.float32), np.array([0]), out_dt=5)
    with pytest.raises(TypeError):
        orc.scatter(np.zeros((1, 4), dtype=np.int32), np.array([0]), np.zeros((4, 4), dtype=np.float32))


# ---- optimizers: independent numpy restatement of the reference's CPU test optimizer -----------
def numpy_reference_step(opt, w, grads_by_row, state, beta12t, lr, wd, eps, b1, b2, alpha, adam_w, dim, padded):
    f = np.float32
    lr, wd, eps, b1, b2, alpha = f(lr), f(wd), f(eps), f(b1), f(b2), f(alpha)
    for row, g in grads_by_row.items():
        g = g.astype(np.float32).copy()
        e = w[row].copy()
        if opt == "adam":
            beta12t[row, 0] = beta12t[row, 0] * b1
            beta12t[row, 1] = beta12t[row, 1] * b2
            b1t, b2t = beta12t[row]
            if adam_w:
                e = e - lr * wd * e
            else:
                g = g + wd * e
            m, v = state[row, :dim].copy(), state[row, padded:padded + dim].copy()
            m = b1 * m + (f(1) - b1) * g
            v = b2 * v + (f(1) - b2) * g * g
            mhat, vhat = m / (f(1) - b1t), v / (f(1) - b2t)
            e = e - lr * mhat / (np.sqrt(vhat) + eps)
            state[row, :dim], state[row, padded:padded + dim] = m, v
        elif opt == "sgd":
            g = g + wd * e
            e = e - lr * g
        elif opt == "adagrad":
            g = g + wd * e
            s = state[row, :dim] + g * g
            e = e - lr * g / (np.sqrt(s) + eps)
            state[row, :dim] = s
        else:
            g = g + wd * e
            v = alpha * state[row, :dim] + (f(1) - alpha) * g * g
            e = e - lr * g / (np.sqrt(v) + eps)
            state[row, :dim] = v
        w[row] = e


@pytest.mark.parametrize("opt,code", [("sgd", 1), ("adam", 2), ("rmsprop", 3), ("adagrad", 4)])
@pytest.mark.parametrize("dim", [3, 32, 129])
@pytest.mark.parametrize("adam_w", [False, True])
def test_optimizers_match_the_numpy_restatement(orc, opt, code, dim, adam_w):
    if adam_w and opt != "adam":
        pytest.skip("decoupled decay exists for Lazy Adam only")
    rows, n, padded = 500, 1_200, -(-dim // 4) * 4
    rng = np.random.default_rng(dim + code)
    w = rng.uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    w2 = w.copy()
    state, state2 = np.zeros((rows, 2 * padded), np.float32), np.zeros((rows, 2 * padded), np.float32)
    beta, beta2 = np.ones((rows, 2), np.float32), np.ones((rows, 2), np.float32)
    hp = dict(lr=0.01, wd=0.05, eps=1e-8, b1=0.9, b2=0.999, alpha=0.99)
    for step in range(3):
        idx = rng.integers(0, rows, size=n).astype(np.int64)
        grads = rng.uniform(-1, 1, size=(n, dim)).astype(np.float32)
        # duplicate sum in arrival order, as the reference's hash-map loop does
        by_row = {}
        for i, r in enumerate(idx):
            by_row[int(r)] = grads[i].copy() if int(r) not in by_row else by_row[int(r)] + grads[i]
        uniq, sums = orc.dedup_gradients(idx, grads)
        assert set(uniq.tolist()) == set(by_row) and np.all(np.diff(uniq) > 0)
        for u, s in zip(uniq, sums):
            assert np.array_equal(s, by_row[int(u)])
        orc.optimizer_apply(code, uniq, sums, w, lr=hp["lr"], state=state, v_offset=padded, beta12t=beta,
                            weight_decay=hp["wd"], epsilon=hp["eps"], beta1=hp["b1"], beta2=hp["b2"],
                            alpha=hp["alpha"], adam_w=adam_w)
        numpy_reference_step(opt, w2, by_row, state2, beta2, hp["lr"], hp["wd"], hp["eps"], hp["b1"], hp["b2"],
                             hp["alpha"], adam_w, dim, padded)
    assert np.array_equal(w, w2) and np.array_equal(state, state2) and np.array_equal(beta, beta2)


def test_bucket_sort_and_distributed_gather_emulation(orc):
    rows, world, dim = 10_007, 4, 16
    off = orc.equal_partition_offsets(rows, world)
    table = np.random.default_rng(0).uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    shards = [table[off[r]:off[r + 1]] for r in range(world)]
    reqs = [np.random.default_rng(10 + r).integers(-3, rows, size=3_000).astype(np.int64) for r in range(world)]
    for r in range(world):
        counts, sorted_ids, raw_pos = orc.bucket_sort_ids(reqs[r], off)
        valid = reqs[r][reqs[r] >= 0]
        assert counts.sum() == valid.size
        assert np.array_equal(np.sort(valid, kind="stable"), sorted_ids[:valid.size])
        assert np.array_equal(reqs[r][raw_pos[:valid.size]], sorted_ids[:valid.size])
        assert np.all(sorted_ids[valid.size:] < 0)                 # negatives sort to the tail
    outs = orc.distributed_gather(shards, off, reqs, out_dt=2)
    for r in range(world):
        want = orc.gather(table, reqs[r], out_dt=2)
        assert np.array_equal(outs[r], want)


def test_round_robin_map_is_the_literal_reference_formula(orc):
    ids = np.arange(0, 64, dtype=np.int64)
    got = orc.round_robin_map(ids, rr=4, world=2, entry_start=100)
    want = 100 + 4 * ((ids // 4) // 2) + ids % 4
    assert np.array_equal(got, want)


def test_two_level_gradient_sum_is_the_single_chain_up_to_rounding(orc):
    """Per-rank sums added in rank order (the order of the distributed gradient apply) against the
    single rank-then-arrival chain and against float64."""
    rng = np.random.default_rng(11)
    ranks, n, dim, rows = 4, 3000, 8, 500
    ids = [rng.integers(0, rows, size=n) for _ in range(ranks)]
    for r in range(ranks):
        ids[r][:400] = 17                                   # longer than a block on every rank
    grads = [rng.normal(0, 1, size=(n, dim)).astype(np.float32) for _ in range(ranks)]
    u2, s2 = orc.dedup_gradients_by_rank(ids, grads, block=256)
    u1, s1 = orc.dedup_gradients(np.concatenate(ids), np.concatenate(grads))
    assert np.array_equal(u1, u2)
    exact = np.zeros((rows, dim))
    np.add.at(exact, np.concatenate(ids), np.concatenate(grads).astype(np.float64))
    scale = np.zeros((rows, dim))
    np.add.at(scale, np.concatenate(ids), np.abs(np.concatenate(grads)).astype(np.float64))
    for s in (s1, s2):                                      # both orders are fp32 sums of the same terms
        assert np.all(np.abs(s - exact[u1]) <= 1e-6 * scale[u1])
    # ids that live on one rank only are summed identically by both orders
    solo_ids = [np.arange(r * 50, r * 50 + 50).repeat(3) for r in range(ranks)]
    solo_g = [rng.normal(0, 1, size=(150, dim)).astype(np.float32) for _ in range(ranks)]
    ua, sa = orc.dedup_gradients_by_rank(solo_ids, solo_g)
    ub, sb = orc.dedup_gradients(np.concatenate(solo_ids), np.concatenate(solo_g))
    assert np.array_equal(ua, ub) and np.array_equal(sa, sb)


def test_cache_policy_model_keeps_the_reference_invariants(orc):
    """What the reference's cache-set tests demand of an update (cacheset_tests.cu:248-276), checked on
    the host model: at most 32 rows per set, lines are distinct, a row that stays keeps its line,
    and no accessed-but-uncached row of a touched set has more accesses than a cached one."""
    rng = np.random.default_rng(5)
    rows, coverage = 64 * 40, 64
    model = orc.CachePolicyModel(rows, coverage)
    for step in range(12):
        hot = rng.integers(0, rows // 8, size=1500)
        ids = np.where(rng.random(1500) < 0.7, hot, rng.integers(0, rows, size=1500))
        before = {s: dict(v) for s, v in model.cached.items()}
        model.update(ids)
        for s in np.unique(ids // coverage):
            lines = model.lines_of(int(s))
            assert 0 < len(lines) <= 32 and len(set(lines.values())) == len(lines)
            assert all(0 <= l < 32 for l in lines.values())
            for r, l in lines.items():
                if r in before.get(int(s), {}):
                    assert before[int(s)][r] == l
            counts = model.count[s * coverage:(s + 1) * coverage]
            cached_min = min(counts[r] for r in lines)
            touched = np.unique(ids[ids // coverage == s]) - s * coverage
            for r in touched:
                if int(r) not in lines:
                    assert counts[r] <= cached_min
    # negative and out-of-range ids are ignored
    total = model.count.sum()
    model.update(np.array([-1, rows, rows + 5]))
    assert model.count.sum() == total


def test_graph_utilities_of_the_oracle(orc):
    """append-unique and self loops on the host: the properties the reference's tests check."""
    rng = np.random.default_rng(2)
    targets = rng.permutation(500)[:60].astype(np.int64)
    neighbors = rng.integers(0, 500, size=2000).astype(np.int64)
    unique, mapping = orc.append_unique(targets, neighbors)
    assert np.array_equal(unique[:60], targets) and len(np.unique(unique)) == len(unique)
    assert set(unique.tolist()) == set(targets.tolist()) | set(neighbors.tolist())
    assert np.array_equal(unique[mapping], neighbors) and mapping.dtype == np.int32
    assert np.all(np.diff(unique[60:]) > 0)
    row_ptr = np.array([0, 2, 2, 5], dtype=np.int32)
    col = np.array([1, 2, 0, 1, 2], dtype=np.int32)
    out_ptr, out_col = orc.csr_add_self_loop(row_ptr, col)
    assert out_ptr.tolist() == [0, 3, 4, 8]
    assert out_col.tolist() == [0, 1, 2, 1, 2, 0, 1, 2]
