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
