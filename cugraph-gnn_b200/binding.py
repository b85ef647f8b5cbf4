"""ctypes binding of libwholegraph.so (the sm_100a build in this package).

The function and class names follow the reference's nanobind module
(python/pylibwholegraph/src/pylibwholegraph/binding/registrations.cpp:288-402) so that code
written against `wholegraph_binding` reads the same here.  Only the C ABI declared in
include/wholegraph/*.h is used; there is no Python or CPU fallback: loading fails loudly when
the shared library is missing.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libwholegraph.so")

MAX_TENSOR_DIM = 8


class ErrorCode(enum.IntEnum):
    SUCCESS = 0
    UNKNOW_ERROR = 1
    NOT_IMPLEMENTED = 2
    LOGIC_ERROR = 3
    CUDA_ERROR = 4
    COMMUNICATION_ERROR = 5
    INVALID_INPUT = 6
    INVALID_VALUE = 7
    OUT_OF_MEMORY = 8
    NOT_SUPPORTED = 9
    SYSTEM_ERROR = 10


class WholeGraphDataType(enum.IntEnum):
    DtUnknown = 0
    DtFloat = 1
    DtHalf = 2
    DtDouble = 3
    DtBF16 = 4
    DtInt = 5
    DtInt64 = 6
    DtInt16 = 7
    DtInt8 = 8
    DtCount = 9


class WholeGraphMemoryType(enum.IntEnum):
    MtNone = 0
    MtContinuous = 1
    MtDistributed = 2
    MtChunked = 3


class WholeGraphMemoryLocation(enum.IntEnum):
    MlNone = 0
    MlDevice = 1
    MlHost = 2


class WholeGraphMemoryAllocType(enum.IntEnum):
    MatNone = 0
    MatDevice = 1
    MatHost = 2
    MatPinned = 3


class WholeGraphOptimizerType(enum.IntEnum):
    OptNone = 0
    OptSgd = 1
    OptLazyAdam = 2
    OptRmsProp = 3
    OptAdaGrad = 4


class WholeGraphAccessType(enum.IntEnum):
    AtNone = 0
    AtReadOnly = 1
    AtReadWrite = 2


class WholeGraphError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = ErrorCode(code)
        super().__init__(f"{what} failed with {self.code.name}")


class TensorDescription(C.Structure):
    _fields_ = [
        ("sizes", C.c_int64 * MAX_TENSOR_DIM),
        ("strides", C.c_int64 * MAX_TENSOR_DIM),
        ("storage_offset", C.c_int64),
        ("dim", C.c_int),
        ("dtype", C.c_int),
    ]


class ArrayDescription(C.Structure):
    """wholegraph_array_description_t"""
    _fields_ = [("size", C.c_int64), ("storage_offset", C.c_int64), ("dtype", C.c_int)]


class MatrixDescription(C.Structure):
    """wholegraph_matrix_description_t"""
    _fields_ = [("sizes", C.c_int64 * 2), ("stride", C.c_int64), ("storage_offset", C.c_int64), ("dtype", C.c_int)]


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


CREATE_CTX_FN = C.CFUNCTYPE(None, C.POINTER(C.c_void_p), C.c_void_p)
DESTROY_CTX_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)
MALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.POINTER(TensorDescription), C.c_int, C.c_void_p, C.c_void_p)
FREE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)


class TempMemoryFns(C.Structure):
    _fields_ = [
        ("create_memory_context_fn", CREATE_CTX_FN),
        ("destroy_memory_context_fn", DESTROY_CTX_FN),
        ("malloc_fn", MALLOC_FN),
        ("free_fn", FREE_FN),
        ("global_context", C.c_void_p),
    ]


class OutputMemoryFns(C.Structure):
    _fields_ = [("malloc_fn", MALLOC_FN), ("free_fn", FREE_FN), ("global_context", C.c_void_p)]


class EnvFns(C.Structure):
    _fields_ = [("temporary_fns", TempMemoryFns), ("output_fns", OutputMemoryFns)]


_lib: Optional[C.CDLL] = None


def _declare(lib: C.CDLL) -> None:
    vp, i64, sz = C.c_void_p, C.c_int64, C.c_size_t
    TD = C.POINTER(TensorDescription)
    sig = {
        "wholegraph_init": (C.c_int, [C.c_uint, C.c_int]),
        "wholegraph_finalize": (C.c_int, []),
        "wholegraph_create_unique_id": (C.c_int, [C.POINTER(UniqueId)]),
        "wholegraph_create_communicator": (C.c_int, [C.POINTER(vp), UniqueId, C.c_int, C.c_int]),
        "wholegraph_split_communicator": (C.c_int, [C.POINTER(vp), vp, C.c_int, C.c_int]),
        "wholegraph_destroy_communicator": (C.c_int, [vp]),
        "wholegraph_communicator_get_rank": (C.c_int, [C.POINTER(C.c_int), vp]),
        "wholegraph_communicator_get_size": (C.c_int, [C.POINTER(C.c_int), vp]),
        "wholegraph_communicator_barrier": (C.c_int, [vp]),
        "wholegraph_communicator_support_type_location": (C.c_int, [vp, C.c_int, C.c_int]),
        "wholegraph_malloc": (C.c_int, [C.POINTER(vp), sz, vp, C.c_int, C.c_int, sz, C.POINTER(sz)]),
        "wholegraph_free": (C.c_int, [vp]),
        "wholegraph_get_memory_type": (C.c_int, [vp]),
        "wholegraph_get_memory_location": (C.c_int, [vp]),
        "wholegraph_get_total_size": (sz, [vp]),
        "wholegraph_get_data_granularity": (sz, [vp]),
        "wholegraph_get_local_memory": (C.c_int, [C.POINTER(vp), C.POINTER(sz), C.POINTER(sz), vp]),
        "wholegraph_get_rank_memory": (C.c_int, [C.POINTER(vp), C.POINTER(sz), C.POINTER(sz), C.c_int, vp]),
        "wholegraph_get_global_pointer": (C.c_int, [C.POINTER(vp), vp]),
        "wholegraph_get_rank_partition_sizes": (C.c_int, [C.POINTER(sz), vp]),
        "wholegraph_get_rank_partition_offsets": (C.c_int, [C.POINTER(sz), vp]),
        "wholegraph_equal_entry_partition_plan": (C.c_int, [C.POINTER(sz), sz, C.c_int]),
        "wholegraph_dtype_get_element_size": (sz, [C.c_int]),
        "wholegraph_initialize_tensor_desc": (None, [TD]),
        "wholegraph_squeeze_tensor": (C.c_bool, [TD, C.c_int]),
        "wholegraph_unsqueeze_tensor": (C.c_bool, [TD, C.c_int]),
        "wholegraph_get_memory_element_count_from_tensor": (i64, [TD]),
        "wholegraph_get_memory_size_from_tensor": (i64, [TD]),
        "wholegraph_create_tensor": (C.c_int, [C.POINTER(vp), TD, vp, C.c_int, C.c_int, C.POINTER(sz)]),
        "wholegraph_destroy_tensor": (C.c_int, [vp]),
        "wholegraph_make_tensor_from_pointer": (C.c_int, [C.POINTER(vp), vp, TD]),
        "wholegraph_make_tensor_from_handle": (C.c_int, [C.POINTER(vp), vp, TD]),
        "wholegraph_tensor_has_handle": (C.c_bool, [vp]),
        "wholegraph_tensor_get_memory_handle": (vp, [vp]),
        "wholegraph_tensor_get_tensor_description": (TD, [vp]),
        "wholegraph_tensor_map_local_tensor": (C.c_int, [vp, C.POINTER(vp)]),
        "wholegraph_tensor_get_data_pointer": (vp, [vp]),
        "wholegraph_tensor_get_entry_offsets": (C.c_int, [C.POINTER(sz), vp]),
        "wholegraph_tensor_get_entry_partition_sizes": (C.c_int, [C.POINTER(sz), vp]),
        "wholegraph_tensor_get_local_entry_count": (C.c_int, [C.POINTER(sz), vp]),
        "wholegraph_tensor_get_local_entry_start": (C.c_int, [C.POINTER(sz), vp]),
        "wholegraph_tensor_get_subtensor": (C.c_int, [vp, C.POINTER(i64), C.POINTER(i64), C.POINTER(vp)]),
        "wholegraph_tensor_get_root": (vp, [vp]),
        "get_wholegraph_tensor_count": (i64, []),
        "wholegraph_gather": (C.c_int, [vp, vp, vp, C.POINTER(EnvFns), vp, C.c_int]),
        "wholegraph_scatter": (C.c_int, [vp, vp, vp, C.POINTER(EnvFns), vp, C.c_int]),
        "wholegraph_b200_get_default_env_func": (C.POINTER(EnvFns), []),
        "wholegraph_b200_get_cached_env_func": (C.POINTER(EnvFns), []),
        "wholegraph_b200_drop_cached_env_func_memory": (None, []),
        "wholegraph_b200_kernel_launch_count": (C.c_ulonglong, []),
        "wholegraph_b200_memcpy_async": (C.c_int, [vp, vp, sz, vp]),
        "wholegraph_b200_partition_workspace_bytes": (sz, [i64, C.c_int]),
        "wholegraph_b200_partition_by_owner": (C.c_int, [vp, C.c_int, i64, C.POINTER(i64), C.c_int, vp, sz,
                                                         vp, vp, vp, vp, vp]),
        "wholegraph_b200_partition_by_owner_no_alloc": (C.c_int, [vp, C.c_int, i64, C.POINTER(i64), C.c_int,
                                                                  vp, vp, vp, vp, vp]),
        "wholegraph_b200_unique_workspace_bytes": (sz, [i64, i64]),
        "wholegraph_b200_unique_by_owner": (C.c_int, [vp, C.c_int, i64, C.POINTER(i64), C.c_int, vp, sz,
                                                      vp, vp, vp, vp, vp]),
        "wholegraph_b200_exchange_chunk_count": (C.c_int, [C.POINTER(i64), C.c_int, sz, C.c_int, C.c_int]),
        "wholegraph_b200_reload_tuning": (C.c_int, [vp]),
        "wholegraph_b200_gather_from_handle": (C.c_int, [vp, vp, vp, vp, vp, vp, C.POINTER(EnvFns), vp, C.c_int]),
        "wholegraph_b200_version": (C.c_char_p, []),
    }
    optional = {
        "wholegraph_create_embedding_optimizer": (C.c_int, [C.POINTER(vp), C.c_int]),
        "wholegraph_optimizer_set_parameter": (C.c_int, [vp, C.c_char_p, vp]),
        "wholegraph_destroy_embedding_optimizer": (None, [vp]),
        "wholegraph_create_embedding_cache_policy": (C.c_int, [C.POINTER(vp), vp, C.c_int, C.c_int, C.c_int, C.c_float]),
        "wholegraph_destroy_embedding_cache_policy": (C.c_int, [vp]),
        "wholegraph_create_embedding": (C.c_int, [C.POINTER(vp), TD, vp, C.c_int, C.c_int, vp, C.POINTER(sz), C.c_int, C.c_int]),
        "wholegraph_destroy_embedding": (C.c_int, [vp]),
        "wholegraph_embedding_get_embedding_tensor": (vp, [vp]),
        "wholegraph_embedding_set_optimizer": (C.c_int, [vp, vp]),
        "wholegraph_embedding_gather": (C.c_int, [vp, vp, vp, C.c_bool, C.POINTER(EnvFns), i64]),
        "wholegraph_embedding_gather_gradient_apply": (C.c_int, [vp, vp, vp, C.c_bool, C.c_float, C.POINTER(EnvFns), i64]),
        "wholegraph_embedding_get_optimizer_state_names": (C.POINTER(C.c_char_p), [vp]),
        "wholegraph_embedding_get_optimizer_state": (vp, [vp, C.c_char_p]),
        "wholegraph_b200_embedding_get_cache_tensors": (C.c_int, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                                                   C.POINTER(C.c_int)]),
        "wholegraph_b200_embedding_get_cache_counters": (C.c_int, [vp, C.POINTER(vp), C.POINTER(i64)]),
        "wholegraph_b200_unique_by_owner_any_order": (C.c_int, [vp, C.c_int, i64, C.POINTER(i64), C.c_int, vp, sz,
                                                                vp, vp, vp, vp, vp]),
        "wholegraph_b200_release_output": (C.c_int, [vp]),
        "graph_append_unique": (C.c_int, [vp, vp, vp, vp, C.POINTER(EnvFns), vp]),
        "csr_add_self_loop": (C.c_int, [vp, vp, vp, vp, vp]),
        "wholegraph_embedding_writeback_cache": (C.c_int, [vp, i64]),
        "wholegraph_embedding_drop_all_cache": (C.c_int, [vp, i64]),
        "wholegraph_load_from_file": (C.c_int, [vp, sz, sz, sz, C.POINTER(C.c_char_p), C.c_int, C.c_int]),
        "wholegraph_store_to_file": (C.c_int, [vp, sz, sz, sz, C.c_char_p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    for name, spec in optional.items():
        if not hasattr(lib, name):
            continue
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = spec


def load_library(path: Optional[str] = None) -> C.CDLL:
    """dlopen libwholegraph.so (RTLD_LOCAL, like the reference's libwholegraph.load_library,
    python/libwholegraph/src/libwholegraph/load.py:38-87)."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(
            f"{p} is missing: build it with `python cugraph-gnn_b200/build.py` "
            "(there is no CPU or Python fallback for the wholegraph ops)")
    lib = C.CDLL(p, mode=C.RTLD_LOCAL)
    _declare(lib)
    if path is None:
        _lib = lib
    return lib


def lib() -> C.CDLL:
    return load_library()


def check(code: int, what: str) -> None:
    if code != 0:
        raise WholeGraphError(code, what)


# --------------------------------------------------------------------------------------------
# thin wrappers, named after the reference's binding functions
# --------------------------------------------------------------------------------------------
def init(flags: int = 0, log_level: int = 3) -> None:
    check(lib().wholegraph_init(flags, log_level), "wholegraph_init")


def finalize() -> None:
    check(lib().wholegraph_finalize(), "wholegraph_finalize")


def create_unique_id() -> UniqueId:
    uid = UniqueId()
    check(lib().wholegraph_create_unique_id(C.byref(uid)), "wholegraph_create_unique_id")
    return uid


def unique_id_to_bytes(uid: UniqueId) -> bytes:
    return C.string_at(C.addressof(uid), C.sizeof(UniqueId))


def unique_id_from_bytes(raw: bytes) -> UniqueId:
    uid = UniqueId()
    C.memmove(C.addressof(uid), raw, C.sizeof(UniqueId))
    return uid


def create_communicator(uid: UniqueId, rank: int, size: int) -> C.c_void_p:
    comm = C.c_void_p()
    check(lib().wholegraph_create_communicator(C.byref(comm), uid, rank, size),
          "wholegraph_create_communicator")
    return comm


def destroy_communicator(comm) -> None:
    check(lib().wholegraph_destroy_communicator(comm), "wholegraph_destroy_communicator")


def make_description(shape: Sequence[int], dtype: WholeGraphDataType,
                     strides: Optional[Sequence[int]] = None, storage_offset: int = 0) -> TensorDescription:
    d = TensorDescription()
    lib().wholegraph_initialize_tensor_desc(C.byref(d))
    d.dim = len(shape)
    d.dtype = int(dtype)
    d.storage_offset = storage_offset
    if strides is None:
        strides, acc = [], 1
        for s in reversed(shape):
            strides.insert(0, acc)
            acc *= max(int(s), 1)
    for i, (s, st) in enumerate(zip(shape, strides)):
        d.sizes[i] = int(s)
        d.strides[i] = int(st)
    return d


def create_wholegraph_tensor(desc: TensorDescription, comm, memory_type, memory_location,
                             entry_partition: Optional[Sequence[int]] = None) -> C.c_void_p:
    t = C.c_void_p()
    part = None
    if entry_partition is not None:
        part = (C.c_size_t * len(entry_partition))(*entry_partition)
    check(lib().wholegraph_create_tensor(C.byref(t), C.byref(desc), comm, int(memory_type),
                                         int(memory_location), part), "wholegraph_create_tensor")
    return t


def make_tensor_from_pointer(ptr: int, desc: TensorDescription) -> C.c_void_p:
    t = C.c_void_p()
    check(lib().wholegraph_make_tensor_from_pointer(C.byref(t), C.c_void_p(ptr), C.byref(desc)),
          "wholegraph_make_tensor_from_pointer")
    return t


def destroy_wholegraph_tensor(t) -> None:
    check(lib().wholegraph_destroy_tensor(t), "wholegraph_destroy_tensor")


def default_env_fns():
    return lib().wholegraph_b200_get_default_env_func()


def cached_env_fns():
    return lib().wholegraph_b200_get_cached_env_func()


def wholegraph_gather_op(wg_tensor, indices, output, env_fns, stream_int: int = 0, gather_sms: int = -1) -> None:
    check(lib().wholegraph_gather(wg_tensor, indices, output, env_fns, C.c_void_p(stream_int), gather_sms),
          "wholegraph_gather")


def wholegraph_scatter_op(input_, indices, wg_tensor, env_fns, stream_int: int = 0, scatter_sms: int = -1) -> None:
    check(lib().wholegraph_scatter(input_, indices, wg_tensor, env_fns, C.c_void_p(stream_int), scatter_sms),
          "wholegraph_scatter")


def local_view(wg_tensor):
    """(pointer, rows) of this rank's shard of a handle tensor."""
    lt = C.c_void_p()
    check(lib().wholegraph_tensor_map_local_tensor(wg_tensor, C.byref(lt)), "wholegraph_tensor_map_local_tensor")
    ptr = lib().wholegraph_tensor_get_data_pointer(lt)
    rows = lib().wholegraph_tensor_get_tensor_description(lt).contents.sizes[0]
    destroy_wholegraph_tensor(lt)
    return ptr, rows


# ---- graph utilities ---------------------------------------------------------------------------
class OutputSlot(C.Structure):
    """wholegraph_b200_output_slot_t: what the built-in output allocator hands back."""
    _fields_ = [("pointer", C.c_void_p), ("description", TensorDescription)]


def append_unique(target_nodes, neighbor_nodes, output_slot, output_neighbor_raw_to_unique_mapping, env_fns,
                  stream_int: int = 0) -> None:
    """Targets followed by the distinct neighbours that are not targets; `output_slot` (an OutputSlot when
    env_fns is one of this library's allocators) receives the list, the optional mapping tensor the position
    of every neighbour in it."""
    check(lib().graph_append_unique(target_nodes, neighbor_nodes, C.byref(output_slot),
                                    output_neighbor_raw_to_unique_mapping, env_fns, C.c_void_p(stream_int)),
          "graph_append_unique")


def release_output(output_slot) -> None:
    """Free the buffer an OutputSlot received from this library's output allocator."""
    check(lib().wholegraph_b200_release_output(C.byref(output_slot)), "wholegraph_b200_release_output")


def add_csr_self_loop(csr_row_ptr, csr_col_ptr, output_csr_row_ptr, output_csr_col_ptr, stream_int: int = 0) -> None:
    check(lib().csr_add_self_loop(csr_row_ptr, csr_col_ptr, output_csr_row_ptr, output_csr_col_ptr,
                                  C.c_void_p(stream_int)), "csr_add_self_loop")


# ---- files ------------------------------------------------------------------------------------
def load_wholegraph_handle_from_filelist(handle, memory_offset: int, memory_entry_size: int, file_entry_size: int,
                                         round_robin_size: int, file_list: Sequence[str]) -> None:
    """Collective: records of `file_entry_size` bytes from the files (taken as one sequence) into slots
    `memory_entry_size` bytes apart, each rank loading its own shard; with round_robin_size > 0 blocks of that
    many records are dealt to the ranks in turn."""
    names = (C.c_char_p * len(file_list))(*[f.encode() for f in file_list])
    check(lib().wholegraph_load_from_file(handle, memory_offset, memory_entry_size, file_entry_size, names,
                                          len(file_list), round_robin_size), "wholegraph_load_from_file")


def store_wholegraph_handle_to_file(handle, memory_offset: int, memory_entry_size: int, file_entry_size: int,
                                    file_name: str) -> None:
    """Collective: every rank writes the records of its shard to its own file."""
    check(lib().wholegraph_store_to_file(handle, memory_offset, memory_entry_size, file_entry_size,
                                         file_name.encode()), "wholegraph_store_to_file")


def tensor_from_filelist(wg_tensor, file_list: Sequence[str], round_robin_size: int = 0) -> None:
    """A 1-D or 2-D handle tensor (or a view of one) filled from files of dense rows."""
    d = lib().wholegraph_tensor_get_tensor_description(wg_tensor).contents
    es = lib().wholegraph_dtype_get_element_size(d.dtype)
    row = es * (d.sizes[1] if d.dim == 2 else 1)
    load_wholegraph_handle_from_filelist(C.c_void_p(lib().wholegraph_tensor_get_memory_handle(wg_tensor)),
                                         d.storage_offset * es, es * d.strides[0], row, round_robin_size, file_list)


def tensor_to_file(wg_tensor, file_name: str) -> None:
    d = lib().wholegraph_tensor_get_tensor_description(wg_tensor).contents
    es = lib().wholegraph_dtype_get_element_size(d.dtype)
    row = es * (d.sizes[1] if d.dim == 2 else 1)
    store_wholegraph_handle_to_file(C.c_void_p(lib().wholegraph_tensor_get_memory_handle(wg_tensor)),
                                    d.storage_offset * es, es * d.strides[0], row, file_name)


# ---- embeddings and sparse optimizers ------------------------------------------------------
def create_embedding(desc: TensorDescription, comm, memory_type, memory_location, cache_policy=None,
                     entry_partition: Optional[Sequence[int]] = None, user_defined_sms: int = -1,
                     round_robin_size: int = 0) -> C.c_void_p:
    e = C.c_void_p()
    part = None
    if entry_partition is not None:
        part = (C.c_size_t * len(entry_partition))(*entry_partition)
    check(lib().wholegraph_create_embedding(C.byref(e), C.byref(desc), comm, int(memory_type),
                                            int(memory_location), cache_policy, part, user_defined_sms,
                                            round_robin_size), "wholegraph_create_embedding")
    return e


def create_cache_policy(cache_comm, memory_type, memory_location, access_type, ratio: float) -> C.c_void_p:
    """A set-associative cache in front of an embedding: `ratio` of the table's rows have a line."""
    p = C.c_void_p()
    check(lib().wholegraph_create_embedding_cache_policy(C.byref(p), cache_comm, int(memory_type),
                                                         int(memory_location), int(access_type), ratio),
          "wholegraph_create_embedding_cache_policy")
    return p


def destroy_cache_policy(policy) -> None:
    check(lib().wholegraph_destroy_embedding_cache_policy(policy), "wholegraph_destroy_embedding_cache_policy")


def embedding_writeback_all_cache(e, stream_int: int = 0) -> None:
    check(lib().wholegraph_embedding_writeback_cache(e, stream_int), "wholegraph_embedding_writeback_cache")


def embedding_drop_all_cache(e, stream_int: int = 0) -> None:
    check(lib().wholegraph_embedding_drop_all_cache(e, stream_int), "wholegraph_embedding_drop_all_cache")


def embedding_cache_tensors(e):
    """(tags, lfu, lines, set coverage) of a cached embedding; the tensors belong to the embedding."""
    tags, lfu, lines, cov = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_int()
    check(lib().wholegraph_b200_embedding_get_cache_tensors(e, C.byref(tags), C.byref(lfu), C.byref(lines),
                                                            C.byref(cov)),
          "wholegraph_b200_embedding_get_cache_tensors")
    return tags, lfu, lines, cov.value


def destroy_embedding(e) -> None:
    check(lib().wholegraph_destroy_embedding(e), "wholegraph_destroy_embedding")


def create_optimizer(opt_type: WholeGraphOptimizerType, **params: float) -> C.c_void_p:
    o = C.c_void_p()
    check(lib().wholegraph_create_embedding_optimizer(C.byref(o), int(opt_type)),
          "wholegraph_create_embedding_optimizer")
    for name, value in params.items():
        v = C.c_float(value)
        check(lib().wholegraph_optimizer_set_parameter(o, name.encode(), C.byref(v)),
              f"wholegraph_optimizer_set_parameter({name})")
    return o


def embedding_tensor(e) -> C.c_void_p:
    return C.c_void_p(lib().wholegraph_embedding_get_embedding_tensor(e))


def embedding_state_names(e) -> list:
    names, arr, i = [], lib().wholegraph_embedding_get_optimizer_state_names(e), 0
    while arr and arr[i] is not None:
        names.append(arr[i].decode())
        i += 1
    return names


def embedding_state(e, name: str) -> C.c_void_p:
    return C.c_void_p(lib().wholegraph_embedding_get_optimizer_state(e, name.encode()))


def EmbeddingGatherForward(e, indices, output, adjust_cache: bool, env_fns, stream_int: int = 0) -> None:
    check(lib().wholegraph_embedding_gather(e, indices, output, adjust_cache, env_fns, stream_int),
          "wholegraph_embedding_gather")


def EmbeddingGatherGradientApply(e, indices, grads, adjust_cache: bool, lr: float, env_fns,
                                 stream_int: int = 0) -> None:
    check(lib().wholegraph_embedding_gather_gradient_apply(e, indices, grads, adjust_cache, lr, env_fns,
                                                           stream_int),
          "wholegraph_embedding_gather_gradient_apply")
