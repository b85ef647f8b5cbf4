"""Descriptor arithmetic, partition planning and optimizer objects of the C ABI (host code only).
Expectations follow the reference's cpp/src/wholegraph/tensor_description.cpp:11-226 and
memory_handle.cpp:1241-1262."""
import ctypes as C

import numpy as np


def test_tensor_description_helpers(wgb):
    lib, DT = wgb.lib(), wgb.WholeGraphDataType
    d = wgb.make_description([100, 32], DT.DtHalf, strides=[40, 1], storage_offset=8)
    assert lib.wholegraph_get_memory_element_count_from_tensor(C.byref(d)) == 4000
    assert lib.wholegraph_get_memory_size_from_tensor(C.byref(d)) == 8000
    # 1-D -> [N, 1] by unsqueeze at the end, as gather does
    a = wgb.make_description([7], DT.DtInt64)
    assert lib.wholegraph_unsqueeze_tensor(C.byref(a), 1)
    assert a.dim == 2 and list(a.sizes[:2]) == [7, 1] and list(a.strides[:2]) == [1, 1]
    assert lib.wholegraph_squeeze_tensor(C.byref(a), 1) and a.dim == 1
    assert not lib.wholegraph_squeeze_tensor(C.byref(a), 0)  # size 7 cannot be squeezed
    # unsqueeze in front takes the displaced axis' stride
    b = wgb.make_description([5, 6], DT.DtFloat)
    assert lib.wholegraph_unsqueeze_tensor(C.byref(b), 0)
    assert list(b.sizes[:3]) == [1, 5, 6] and list(b.strides[:3]) == [6, 6, 1]
    z = wgb.TensorDescription()
    lib.wholegraph_initialize_tensor_desc(C.byref(z))
    assert z.dim == 0 and z.dtype == 0 and all(s == 1 for s in z.sizes) and all(s == 1 for s in z.strides)
    assert lib.wholegraph_get_memory_element_count_from_tensor(C.byref(z)) == 1


def test_equal_partition_plan_matches_the_oracle(wgb, orc):
    lib = wgb.lib()
    for rows, world in [(10, 3), (100_000_000, 8), (7, 8), (1, 1), (240_000_000, 8), (13, 2)]:
        per = C.c_size_t()
        assert lib.wholegraph_equal_entry_partition_plan(C.byref(per), rows, world) == 0
        off = orc.equal_partition_offsets(rows, world)
        assert per.value == -(-rows // world)
        want = np.minimum(np.arange(world + 1) * per.value, rows)
        assert np.array_equal(off, want)
        # owner rule: last rank whose first row is <= id
        for rid in (0, rows - 1, rows // 2):
            owner = orc.lib().wgo_owner(rid, C.c_void_p(off.ctypes.data), world)
            assert off[owner] <= rid < max(off[owner + 1], rid + 1)
            assert owner == min(rid // per.value, world - 1)


def test_optimizer_objects(wgb):
    lib = wgb.lib()
    for opt, ok, bad in [(wgb.WholeGraphOptimizerType.OptSgd, ["weight_decay"], ["epsilon", "lr"]),
                         (wgb.WholeGraphOptimizerType.OptLazyAdam, ["weight_decay", "epsilon", "beta1", "beta2", "adam_w"], ["alpha"]),
                         (wgb.WholeGraphOptimizerType.OptAdaGrad, ["weight_decay", "epsilon"], ["beta1"]),
                         (wgb.WholeGraphOptimizerType.OptRmsProp, ["weight_decay", "epsilon", "alpha"], ["beta2"])]:
        o = wgb.create_optimizer(opt)
        v = C.c_float(0.25)
        for name in ok:
            assert lib.wholegraph_optimizer_set_parameter(o, name.encode(), C.byref(v)) == 0
        for name in bad:
            assert lib.wholegraph_optimizer_set_parameter(o, name.encode(), C.byref(v)) == int(wgb.ErrorCode.INVALID_INPUT)
        lib.wholegraph_destroy_embedding_optimizer(o)
    o = C.c_void_p()
    assert lib.wholegraph_create_embedding_optimizer(C.byref(o), 0) == int(wgb.ErrorCode.NOT_IMPLEMENTED)


def test_cache_policy_ratio_bounds(wgb):
    lib = wgb.lib()
    p = C.c_void_p()
    assert lib.wholegraph_create_embedding_cache_policy(C.byref(p), None, 1, 1, 1, C.c_float(0.001)) == int(wgb.ErrorCode.INVALID_VALUE)
    assert lib.wholegraph_create_embedding_cache_policy(C.byref(p), None, 1, 1, 1, C.c_float(1.5)) == int(wgb.ErrorCode.INVALID_VALUE)
    assert lib.wholegraph_create_embedding_cache_policy(C.byref(p), None, 1, 1, 1, C.c_float(0.1)) == 0
    assert lib.wholegraph_destroy_embedding_cache_policy(p) == 0


def _fake_tensor(wgb, sizes, dtype, address=0x10000):
    """A descriptor-only tensor over an address that is never dereferenced: argument checks only."""
    return wgb.make_tensor_from_pointer(address, wgb.make_description(sizes, dtype))


def test_graph_utilities_check_their_arguments_before_any_device_work(wgb):
    lib, DT, E = wgb.lib(), wgb.WholeGraphDataType, wgb.ErrorCode
    i32 = _fake_tensor(wgb, [8], DT.DtInt)
    i64 = _fake_tensor(wgb, [8], DT.DtInt64)
    f32 = _fake_tensor(wgb, [8], DT.DtFloat)
    m2d = _fake_tensor(wgb, [4, 2], DT.DtInt)
    env = wgb.default_env_fns() if hasattr(wgb, "default_env_fns") else wgb.cached_env_fns()
    slot = wgb.OutputSlot()
    # append unique: 1-D ids of one integer type, int32 mapping
    assert lib.graph_append_unique(m2d, i32, C.byref(slot), None, env, None) == int(E.INVALID_INPUT)
    assert lib.graph_append_unique(i32, m2d, C.byref(slot), None, env, None) == int(E.INVALID_INPUT)
    assert lib.graph_append_unique(i32, i64, C.byref(slot), None, env, None) == int(E.LOGIC_ERROR)
    assert lib.graph_append_unique(f32, f32, C.byref(slot), None, env, None) == int(E.INVALID_INPUT)
    assert lib.graph_append_unique(i64, i64, C.byref(slot), i64, env, None) == int(E.INVALID_INPUT)   # mapping not int32
    assert lib.graph_append_unique(None, i64, C.byref(slot), None, env, None) == int(E.INVALID_INPUT)
    assert slot.pointer is None
    # self loops: four 1-D int32 tensors, outputs large enough
    small = _fake_tensor(wgb, [3], DT.DtInt)
    assert lib.csr_add_self_loop(i64, i32, i32, i32, None) == int(E.INVALID_INPUT)
    assert lib.csr_add_self_loop(i32, m2d, i32, i32, None) == int(E.INVALID_INPUT)
    assert lib.csr_add_self_loop(i32, i32, small, i32, None) == int(E.INVALID_INPUT)                  # 8 row pointers need 8
    assert lib.csr_add_self_loop(i32, i32, i32, i32, None) == int(E.INVALID_INPUT)                    # 8 + 7 columns needed
    for t in (i32, i64, f32, m2d, small):
        wgb.destroy_wholegraph_tensor(t)
    assert lib.wholegraph_b200_release_output(None) == int(E.INVALID_INPUT)
    assert lib.wholegraph_b200_release_output(C.byref(slot)) == 0                                      # empty slot: nothing to free


def test_sampling_entry_points_refuse(wgb):
    lib = wgb.lib()
    for name in ("wholegraph_csr_unweighted_sample_without_replacement", "wholegraph_csr_weighted_sample_without_replacement",
                 "generate_random_positive_int_cpu", "generate_exponential_distribution_negative_float_cpu"):
        assert hasattr(lib, name)
    lib.generate_random_positive_int_cpu.argtypes = [C.c_int64, C.c_int64, C.c_void_p]
    assert lib.generate_random_positive_int_cpu(1, 0, None) == int(wgb.ErrorCode.NOT_IMPLEMENTED)


def _chunk_count(wgb, matrix, row_bytes, wanted=0, forced=0):
    m = np.ascontiguousarray(matrix, dtype=np.int64)
    return wgb.lib().wholegraph_b200_exchange_chunk_count(
        m.ctypes.data_as(C.POINTER(C.c_int64)), m.shape[0], row_bytes, wanted, forced)


def test_exchange_chunk_count_depends_only_on_the_count_matrix(wgb):
    """Every chunk of a pipelined exchange is a matched set of NCCL sends and receives, so all ranks
    must pick the same number of chunks.  The choice is a function of the world x world count
    matrix alone: an asymmetric exchange with ranks on either side of the 16 MiB threshold still
    gives one answer, the busiest rank's."""
    row_bytes, threshold_rows = 256, (16 << 20) // 256
    # rank 0 sends far more than the threshold, the others far less: one K for everybody
    m = np.array([[5, threshold_rows * 3, 10], [7, 0, 3], [1, 2, 9]])
    assert _chunk_count(wgb, m, row_bytes) == 4
    assert _chunk_count(wgb, m.T, row_bytes) == 4                 # the receive side counts as well
    # just below / just at the threshold on the busiest rank; the diagonal (own rows) never counts
    below = np.array([[10 ** 9, threshold_rows - 1], [0, 10 ** 9]])
    assert _chunk_count(wgb, below, row_bytes) == 1
    at = np.array([[0, threshold_rows], [0, 0]])
    assert _chunk_count(wgb, at, row_bytes) == 4
    # a caller's wish and the environment override, both capped
    assert _chunk_count(wgb, m, row_bytes, wanted=1) == 1
    assert _chunk_count(wgb, m, row_bytes, wanted=1, forced=8) == 8
    assert _chunk_count(wgb, m, row_bytes, wanted=99) == 16
    # what the old rule did wrong: a per-rank answer.  Rank by rank, the outgoing bytes differ ...
    out_bytes = [(m[q].sum() - m[q, q]) * row_bytes for q in range(3)]
    assert out_bytes[0] >= 16 << 20 > out_bytes[1]
    # ... yet the matrix every rank holds gives the same K whichever rank evaluates it.
    assert len({_chunk_count(wgb, m.copy(), row_bytes) for _ in range(3)}) == 1


def test_partition_entry_points_reject_a_bad_owner_table(wgb):
    """first_row must start at 0 and must not decrease: the kernels walk it from an estimate and
    would leave the table otherwise.  Both entry points refuse before anything is launched (the
    pointers below are never dereferenced)."""
    lib, E = wgb.lib(), wgb.ErrorCode
    fake = C.c_void_p(0x10000)
    for table in ([5, 10, 20], [0, 12, 8], [0, 10, 5, 20]):
        world = len(table) - 1
        fr = (C.c_int64 * len(table))(*table)
        rc = lib.wholegraph_b200_partition_by_owner(fake, 1, 100, fr, world, fake, 1 << 20, fake, fake, fake, fake, None)
        assert rc == int(E.INVALID_VALUE), table
        rc = lib.wholegraph_b200_partition_by_owner_no_alloc(fake, 1, 100, fr, world, fake, fake, fake, fake, None)
        assert rc == int(E.INVALID_VALUE), table
        rc = lib.wholegraph_b200_unique_by_owner(fake, 1, 100, fr, world, fake, 1 << 30, fake, fake, fake, fake, None)
        assert rc == int(E.INVALID_VALUE), table
    ok = (C.c_int64 * 3)(0, 10, 20)
    assert lib.wholegraph_b200_partition_by_owner(fake, 1, 100, ok, 2, fake, 0, fake, fake, fake, fake, None) == int(E.INVALID_VALUE)  # workspace too small
    assert lib.wholegraph_b200_unique_by_owner(fake, 1, 100, ok, 2, fake, 0, fake, fake, fake, fake, None) == int(E.INVALID_VALUE)
    assert lib.wholegraph_b200_unique_by_owner(None, 1, 100, ok, 2, fake, 1 << 30, fake, fake, fake, fake, None) == int(E.INVALID_INPUT)
