"""numpy front end of the CPU oracle (oracle/wg_oracle.c).  TEST INFRASTRUCTURE ONLY.

Every function restates one step of the reference's hot path; see the C file for the
reference file:line each one follows.  Arrays are numpy; fp16 is np.float16, bf16 travels as
np.uint16 bit patterns (numpy has no bfloat16).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

# wholegraph_dtype_t codes
DT_FLOAT, DT_HALF, DT_DOUBLE, DT_BF16, DT_INT, DT_INT64, DT_INT16, DT_INT8 = 1, 2, 3, 4, 5, 6, 7, 8
OPT_SGD, OPT_LAZY_ADAM, OPT_RMSPROP, OPT_ADAGRAD = 1, 2, 3, 4

_NP = {DT_FLOAT: np.float32, DT_HALF: np.float16, DT_DOUBLE: np.float64, DT_BF16: np.uint16,
       DT_INT: np.int32, DT_INT64: np.int64, DT_INT16: np.int16, DT_INT8: np.int8}


def np_dtype(dt: int):
    return np.dtype(_NP[dt])


def wg_dtype(a: np.ndarray, bf16: bool = False) -> int:
    if bf16:
        assert a.dtype == np.uint16
        return DT_BF16
    for k, v in _NP.items():
        if k != DT_BF16 and a.dtype == np.dtype(v):
            return k
    raise TypeError(f"no wholegraph dtype for {a.dtype}")


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        src = os.path.join(_HERE, "wg_oracle.c")
        if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
            subprocess.run(["make", "-s", "-C", _HERE], check=True)
        _lib = C.CDLL(_LIB_PATH)
        i64, vp, ci = C.c_int64, C.c_void_p, C.c_int
        _lib.wgo_gather.restype = ci
        _lib.wgo_gather.argtypes = [vp, ci, i64, i64, i64, vp, ci, i64, vp, vp, ci, i64, i64, ci]
        _lib.wgo_scatter.restype = ci
        _lib.wgo_scatter.argtypes = [vp, ci, i64, i64, i64, vp, ci, i64, vp, ci, i64, i64, ci]
        _lib.wgo_equal_partition_offsets.restype = None
        _lib.wgo_equal_partition_offsets.argtypes = [i64, ci, vp]
        _lib.wgo_owner.restype = ci
        _lib.wgo_owner.argtypes = [i64, vp, ci]
        _lib.wgo_bucket_sort_ids.restype = ci
        _lib.wgo_bucket_sort_ids.argtypes = [vp, ci, i64, vp, ci, vp, vp, vp]
        _lib.wgo_dedup_gradients_blocked.restype = i64
        _lib.wgo_dedup_gradients_blocked.argtypes = [vp, ci, i64, vp, ci, i64, i64, i64, vp, vp]
        _lib.wgo_optimizer_apply.restype = ci
        _lib.wgo_optimizer_apply.argtypes = [ci, vp, i64, vp, i64, i64, vp, ci, i64, vp, i64, i64, vp, i64,
                                             C.c_float, C.c_float, C.c_float, C.c_float, C.c_float,
                                             C.c_float, ci, ci]
        _lib.wgo_round_robin_map.restype = None
        _lib.wgo_round_robin_map.argtypes = [vp, ci, i64, i64, ci, i64, vp]
        _lib.wgo_float_to_half.restype = C.c_uint16
        _lib.wgo_float_to_half.argtypes = [C.c_float]
        _lib.wgo_float_to_bf16.restype = C.c_uint16
        _lib.wgo_float_to_bf16.argtypes = [C.c_float]
        _lib.wgo_half_to_float.restype = C.c_float
        _lib.wgo_half_to_float.argtypes = [C.c_uint16]
        _lib.wgo_bf16_to_float.restype = C.c_float
        _lib.wgo_bf16_to_float.argtypes = [C.c_uint16]
    return _lib


def _p(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


def _idx_dt(idx: np.ndarray) -> int:
    if idx.dtype == np.int32:
        return DT_INT
    if idx.dtype == np.int64:
        return DT_INT64
    raise TypeError("indices must be int32 or int64")


def _matrix_params(a: np.ndarray):
    """(dim, row stride in elements) of a C-contiguous-per-row 1-D / 2-D array."""
    if a.size == 0:  # numpy reports arbitrary strides for empty arrays
        return (1, 1) if a.ndim == 1 else (a.shape[1], max(a.shape[1], 1))
    if a.ndim == 1:
        assert a.strides[0] == a.itemsize
        return 1, 1
    assert a.ndim == 2 and a.strides[1] == a.itemsize and a.strides[0] % a.itemsize == 0
    return a.shape[1], a.strides[0] // a.itemsize


def gather(table: np.ndarray, indices: np.ndarray, out_dt: int | None = None, out: np.ndarray | None = None,
           table_bf16: bool = False, raw_pos: np.ndarray | None = None, threads: int = 1) -> np.ndarray:
    """out[i] = cast(table[indices[i]]), rows with a negative index left as they are.

    `table` / `out` may be row-strided views (ndarray slices); bf16 data is uint16 bit patterns
    (pass table_bf16 / out_dt=DT_BF16).
    """
    tab_dt = wg_dtype(table, table_bf16)
    dim, tstride = _matrix_params(table)
    if out_dt is None:
        out_dt = tab_dt
    n = indices.shape[0]
    if out is None:
        shape = (n,) if table.ndim == 1 else (n, dim)
        out = np.zeros(shape, dtype=np_dtype(out_dt))
    odim, ostride = _matrix_params(out)
    assert odim == dim and (raw_pos is not None or out.shape[0] == n)
    indices = np.ascontiguousarray(indices)
    rp = None
    if raw_pos is not None:
        rp = np.ascontiguousarray(raw_pos, dtype=np.int64)
    rc = lib().wgo_gather(_p(table), tab_dt, dim, tstride, 0, _p(indices), _idx_dt(indices), n,
                          _p(rp) if rp is not None else None, _p(out), out_dt, ostride, 0, threads)
    if rc != 0:
        raise TypeError("gather between floating point and integer dtypes is not allowed")
    return out


def scatter(rows: np.ndarray, indices: np.ndarray, table: np.ndarray, rows_bf16: bool = False,
            table_bf16: bool = False, threads: int = 1) -> np.ndarray:
    """table[indices[i]] = cast(rows[i]) in place; negative indices are skipped."""
    in_dt, tab_dt = wg_dtype(rows, rows_bf16), wg_dtype(table, table_bf16)
    dim, istride = _matrix_params(rows)
    tdim, tstride = _matrix_params(table)
    assert dim == tdim and rows.shape[0] == indices.shape[0]
    indices = np.ascontiguousarray(indices)
    rc = lib().wgo_scatter(_p(rows), in_dt, dim, istride, 0, _p(indices), _idx_dt(indices), indices.shape[0],
                           _p(table), tab_dt, tstride, 0, threads)
    if rc != 0:
        raise TypeError("scatter between floating point and integer dtypes is not allowed")
    return table


def equal_partition_offsets(rows: int, world: int) -> np.ndarray:
    off = np.zeros(world + 1, dtype=np.int64)
    lib().wgo_equal_partition_offsets(rows, world, _p(off))
    return off


def bucket_sort_ids(indices: np.ndarray, offsets: np.ndarray):
    """(counts[W], sorted_ids[n], raw_pos[n]) of one rank's request list."""
    indices = np.ascontiguousarray(indices)
    offsets = np.ascontiguousarray(offsets, dtype=np.int64)
    world = offsets.shape[0] - 1
    n = indices.shape[0]
    counts = np.zeros(world, dtype=np.int64)
    sorted_ids = np.zeros(n, dtype=np.int64)
    raw_pos = np.zeros(n, dtype=np.int64)
    rc = lib().wgo_bucket_sort_ids(_p(indices), _idx_dt(indices), n, _p(offsets), world, _p(counts),
                                   _p(sorted_ids), _p(raw_pos))
    assert rc == 0
    return counts, sorted_ids, raw_pos


def dedup_gradients(indices: np.ndarray, grads: np.ndarray, grads_bf16: bool = False, block: int = 0):
    """(unique ids, fp32 sums) with duplicates added in arrival order (block = 0: one chain per
    id, the reference's order; block > 0: runs longer than `block` summed block by block)."""
    indices = np.ascontiguousarray(indices)
    dim, gstride = _matrix_params(grads)
    n = indices.shape[0]
    uniq = np.zeros(n, dtype=np.int64)
    sums = np.zeros((max(n, 1), dim), dtype=np.float32)
    u = lib().wgo_dedup_gradients_blocked(_p(indices), _idx_dt(indices), n, _p(grads), wg_dtype(grads, grads_bf16),
                                          dim, gstride, block, _p(uniq), _p(sums))
    assert u >= 0
    return uniq[:u].copy(), sums[:u].copy()


def dedup_gradients_by_rank(rank_indices, rank_grads, block: int = 256):
    """Two-level order of the distributed gradient apply when every rank pre-sums its own
    duplicates: per rank, duplicates are added in arrival order (runs longer than `block` block by
    block); the owner then adds the per-rank sums of an id in rank order.  Returns (unique ids,
    fp32 sums) over all ranks."""
    ids, sums = [], []
    for idx, g in zip(rank_indices, rank_grads):
        u, s = dedup_gradients(idx, g, block=block)
        ids.append(u)
        sums.append(s)
    return dedup_gradients(np.concatenate(ids), np.concatenate(sums), block=block)


def optimizer_apply(opt: int, ids: np.ndarray, grads: np.ndarray, weights: np.ndarray, *, lr: float,
                    state: np.ndarray | None = None, v_offset: int = 0, beta12t: np.ndarray | None = None,
                    local_start: int = 0, weight_decay: float = 0.0, epsilon: float = 1e-8,
                    beta1: float = 0.9, beta2: float = 0.999, alpha: float = 0.99, adam_w: bool = False,
                    weights_bf16: bool = False, threads: int = 1) -> None:
    """One sparse optimizer step on unique `ids` (in place on weights / state / beta12t)."""
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    assert grads.dtype == np.float32
    dim, gstride = _matrix_params(grads)
    _, wstride = _matrix_params(weights)
    sstride = 0
    if state is not None:
        assert state.dtype == np.float32
        _, sstride = _matrix_params(state)
    if beta12t is not None:
        assert beta12t.dtype == np.float32 and beta12t.flags.c_contiguous
    rc = lib().wgo_optimizer_apply(opt, _p(ids), ids.shape[0], _p(grads), dim, gstride, _p(weights),
                                   wg_dtype(weights, weights_bf16), wstride,
                                   _p(state) if state is not None else None, sstride, v_offset,
                                   _p(beta12t) if beta12t is not None else None, local_start, lr,
                                   weight_decay, epsilon, beta1, beta2, alpha, 1 if adam_w else 0, threads)
    assert rc == 0


def round_robin_map(indices: np.ndarray, rr: int, world: int, entry_start: int) -> np.ndarray:
    indices = np.ascontiguousarray(indices)
    out = np.zeros_like(indices)
    lib().wgo_round_robin_map(_p(indices), _idx_dt(indices), indices.shape[0], rr, world, entry_start, _p(out))
    return out


def float_to_half_bits(x: np.ndarray) -> np.ndarray:
    f = lib().wgo_float_to_half
    return np.array([f(float(v)) for v in np.asarray(x, dtype=np.float32).ravel()], dtype=np.uint16)


def float_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(x.shape, dtype=np.uint16)
    t = x.reshape(-1, 1) if x.ndim != 2 else x
    o = out.reshape(t.shape)
    gather(t, np.arange(t.shape[0], dtype=np.int64), out_dt=DT_BF16, out=o)
    return out


def bf16_bits_to_float(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- composed multi-rank paths (all ranks emulated in one process) -------------------------
def distributed_gather(shards: list[np.ndarray], offsets: np.ndarray, requests: list[np.ndarray], out_dt: int,
                       shards_bf16: bool = False) -> list[np.ndarray]:
    """What every rank's output holds after a DISTRIBUTED gather: bucket + sort the ids, serve
    them from the owners' shards with the cast to the output dtype done at the owner, send the
    rows back and reorder them (reference: gather_op_impl_nccl.cu:23-171)."""
    world = len(shards)
    dim = shards[0].shape[1]
    plans = [bucket_sort_ids(r, offsets) for r in requests]
    outs = []
    for rank in range(world):
        counts, sorted_ids, raw_pos = plans[rank]
        out = np.zeros((requests[rank].shape[0], dim), dtype=np_dtype(out_dt))
        start = 0
        for owner in range(world):
            c = int(counts[owner])
            ids_local = sorted_ids[start:start + c] - offsets[owner]
            rows = gather(shards[owner], ids_local, out_dt=out_dt, table_bf16=shards_bf16)
            # reorder: received row j goes to output row raw_pos[start + j]
            out[raw_pos[start:start + c]] = rows
            start += c
        outs.append(out)
    return outs


class CachePolicyModel:
    """Set-associative embedding cache, restated on the host: which rows of a table hold one of the
    32 lines of their set after a sequence of access batches.

    Geometry is the reference's (cpp/src/wholegraph/embedding_cache.hpp:64-74: sets of 32 lines,
    a set covers `coverage` consecutive rows).  The replacement rule is the one this repository's
    update kernel states, which satisfies what the reference's cache-set tests check
    (cpp/tests/wholegraph_tensor_ops/cacheset_tests.cu:248-276: after an update no uncached row of
    a touched set has a higher access count than a cached one; which of equal-count rows stay is
    free): counters are exact; after a batch the cached rows of every touched set are the 32 with
    the highest counters among (cached U accessed), cached rows first on ties, then lower row
    numbers; rows that stay keep their line, new rows take the freed lines in priority order."""

    SET_SIZE = 32

    def __init__(self, rows: int, coverage: int):
        assert rows % coverage == 0 and coverage >= self.SET_SIZE
        self.count = np.zeros(rows, dtype=np.int64)
        self.coverage = coverage
        self.cached = {}          # set -> {row in set: line}

    def update(self, ids: np.ndarray) -> None:
        ids = np.asarray(ids, dtype=np.int64)
        ids = ids[(ids >= 0) & (ids < self.count.shape[0])]
        uniq, cnt = np.unique(ids, return_counts=True)
        self.count[uniq] += cnt
        for s in np.unique(uniq // self.coverage):
            s = int(s)
            lines = self.cached.setdefault(s, {})
            touched = uniq[uniq // self.coverage == s] - s * self.coverage
            cand = [(-(int(self.count[s * self.coverage + r]) * 2 + 1), int(r)) for r in lines]
            cand += [(-(int(self.count[s * self.coverage + r]) * 2), int(r)) for r in touched if int(r) not in lines]
            keep = [r for _, r in sorted(cand)[: self.SET_SIZE]]
            free = sorted(set(range(self.SET_SIZE)) - {lines[r] for r in keep if r in lines})
            new = {r: lines[r] for r in keep if r in lines}
            for r in keep:
                if r not in lines:
                    new[r] = free.pop(0)
            self.cached[s] = new

    def lines_of(self, s: int) -> dict:
        return self.cached.get(s, {})


def append_unique(targets: np.ndarray, neighbors: np.ndarray):
    """(unique nodes, mapping) of the append-unique step: the targets in their order, then every
    distinct neighbour that is not a target, ascending; mapping[j] = position of neighbors[j] in
    that list (a neighbour equal to several targets maps to the first of them).

    The reference guarantees the same except for the order of the appended neighbours, which is the
    order of its hash table (cpp/src/graph_ops/append_unique_func.cuh:263-341)."""
    targets, neighbors = np.asarray(targets), np.asarray(neighbors)
    first = {}
    for i, t in enumerate(targets.tolist()):
        first.setdefault(t, i)
    new = sorted(set(neighbors.tolist()) - set(first))
    where = dict(first)
    where.update({v: len(targets) + k for k, v in enumerate(new)})
    unique = np.concatenate([targets, np.asarray(new, dtype=targets.dtype)]) if len(new) else targets.copy()
    mapping = np.asarray([where[v] for v in neighbors.tolist()], dtype=np.int32)
    return unique, mapping


def csr_add_self_loop(row_ptr: np.ndarray, col: np.ndarray):
    """CSR with edge (r, r) put first in every row (cpp/src/graph_ops/csr_add_self_loop_func.cuh:13-32)."""
    row_ptr, col = np.asarray(row_ptr, dtype=np.int32), np.asarray(col, dtype=np.int32)
    rows = len(row_ptr) - 1
    out_ptr = (row_ptr + np.arange(rows + 1, dtype=np.int32)).astype(np.int32)
    out_col = np.empty(len(col) + rows, dtype=np.int32)
    for r in range(rows):
        out_col[out_ptr[r]] = r
        out_col[out_ptr[r] + 1:out_ptr[r + 1]] = col[row_ptr[r]:row_ptr[r + 1]]
    return out_ptr, out_col
