"""torch <-> wholegraph glue: dtype maps, tensor wrapping, views of device shards.

torch is used for device memory and streams only; every op goes through the C ABI.
Mirrors the helpers of the reference's torch adapter
(python/wholegraph-torch/src/wholegraph_torch/utils.py, wholegraph_env.py:19-26).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import binding as wgb
from .binding import WholeGraphDataType as DT

TORCH_TO_WG = {
    torch.float32: DT.DtFloat,
    torch.float16: DT.DtHalf,
    torch.float64: DT.DtDouble,
    torch.bfloat16: DT.DtBF16,
    torch.int32: DT.DtInt,
    torch.int64: DT.DtInt64,
    torch.int16: DT.DtInt16,
    torch.int8: DT.DtInt8,
}
WG_TO_TORCH = {v: k for k, v in TORCH_TO_WG.items()}
_TYPESTR = {
    torch.float32: "<f4", torch.float16: "<f2", torch.float64: "<f8", torch.int32: "<i4",
    torch.int64: "<i8", torch.int16: "<i2", torch.int8: "|i1", torch.bfloat16: "<i2",
}


def current_stream_int() -> int:
    return torch.cuda.current_stream().cuda_stream


def wrap_torch_tensor(t: torch.Tensor):
    """Non-owning wholegraph tensor over a 1-D / 2-D torch tensor (inner stride 1).

    The storage pointer handed over is the tensor's data pointer, so storage_offset is 0 and
    the row stride is the torch stride (role of WrappedLocalTensor.wrap_tensor).
    """
    if t.dim() not in (1, 2):
        raise ValueError("need a 1-D or 2-D tensor")
    strides = list(t.stride())
    if t.numel() == 0:  # torch reports arbitrary strides for empty tensors
        strides = [t.shape[1], 1] if t.dim() == 2 else [1]
    if strides[-1] != 1:
        raise ValueError("need a tensor with unit inner stride")
    desc = wgb.make_description(list(t.shape), TORCH_TO_WG[t.dtype], strides=strides)
    return wgb.make_tensor_from_pointer(t.data_ptr(), desc)


class _DevicePointerView:
    """Minimal __cuda_array_interface__ carrier for memory owned by a wholegraph handle."""

    def __init__(self, ptr: int, shape, dtype: torch.dtype, strides_elems=None, owner=None):
        itemsize = torch.empty((), dtype=dtype).element_size()
        iface = {
            "shape": tuple(int(s) for s in shape),
            "typestr": _TYPESTR[dtype],
            "data": (int(ptr), False),
            "version": 3,
        }
        if strides_elems is not None:
            iface["strides"] = tuple(int(s) * itemsize for s in strides_elems)
        self.__cuda_array_interface__ = iface
        self._owner = owner


def view_device_memory(ptr: int, shape, dtype: torch.dtype, strides_elems=None, device=None) -> torch.Tensor:
    """torch view of `ptr` (no copy).  bf16 goes through an int16 view."""
    if 0 in tuple(shape):
        return torch.empty(tuple(shape), dtype=dtype, device=device or "cuda")
    base = torch.as_tensor(_DevicePointerView(ptr, shape, dtype, strides_elems), device=device or "cuda")
    return base.view(torch.bfloat16) if dtype == torch.bfloat16 else base


def local_shard_as_torch(wg_tensor) -> torch.Tensor:
    """This rank's rows of a handle tensor as a torch tensor sharing the memory."""
    lib = wgb.lib()
    lt = C.c_void_p()
    wgb.check(lib.wholegraph_tensor_map_local_tensor(wg_tensor, C.byref(lt)), "map_local_tensor")
    try:
        d = lib.wholegraph_tensor_get_tensor_description(lt).contents
        ptr = lib.wholegraph_tensor_get_data_pointer(lt)
        dtype = WG_TO_TORCH[DT(d.dtype)]
        shape = [d.sizes[i] for i in range(d.dim)]
        strides = [d.strides[i] for i in range(d.dim)]
    finally:
        wgb.destroy_wholegraph_tensor(lt)
    return view_device_memory(ptr or 0, shape, dtype, strides)


def write_local_shard(wg_tensor, rows: torch.Tensor, first_local_row: int = 0) -> None:
    """Copy `rows` (contiguous, same dtype and row width as the table's storage rows) into this
    rank's shard starting at local row `first_local_row`, on the current stream.  Goes through the
    C ABI with raw pointers, so it also works where the shard cannot be viewed as a torch tensor."""
    lib = wgb.lib()
    lt = C.c_void_p()
    wgb.check(lib.wholegraph_tensor_map_local_tensor(wg_tensor, C.byref(lt)), "map_local_tensor")
    try:
        d = lib.wholegraph_tensor_get_tensor_description(lt).contents
        ptr = lib.wholegraph_tensor_get_data_pointer(lt)
        stride = d.strides[0] if d.dim == 2 else 1
        width = d.sizes[1] if d.dim == 2 else 1
        local_rows = d.sizes[0]
    finally:
        wgb.destroy_wholegraph_tensor(lt)
    if rows.numel() == 0:
        return
    if not rows.is_contiguous() or TORCH_TO_WG[rows.dtype] != DT(d.dtype):
        raise ValueError("rows must be contiguous and of the table dtype")
    if stride != width or (rows.dim() == 2 and rows.shape[1] != width):
        raise ValueError("write_local_shard needs densely packed rows")
    if first_local_row + rows.shape[0] > local_rows:
        raise ValueError("rows exceed the local shard")
    nbytes = rows.numel() * rows.element_size()
    dst = ptr + first_local_row * stride * rows.element_size()
    wgb.check(lib.wholegraph_b200_memcpy_async(C.c_void_p(dst), C.c_void_p(rows.data_ptr()), nbytes,
                                               C.c_void_p(current_stream_int())), "memcpy_async")


def gather(wg_table, indices: torch.Tensor, out: torch.Tensor, env=None, sms: int = -1) -> torch.Tensor:
    """out[i] = cast(table[indices[i]]) on the current stream (role of WholeGraphTensor.gather,
    python/wholegraph-torch/src/wholegraph_torch/tensor.py:52-73)."""
    wi, wo = wrap_torch_tensor(indices), wrap_torch_tensor(out)
    try:
        wgb.wholegraph_gather_op(wg_table, wi, wo, env or wgb.cached_env_fns(), current_stream_int(), sms)
    finally:
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wo)
    return out


def scatter(inp: torch.Tensor, indices: torch.Tensor, wg_table, env=None, sms: int = -1) -> None:
    """table[indices[i]] = cast(inp[i]) on the current stream (role of WholeGraphTensor.scatter,
    tensor.py:75-90)."""
    wi, wn = wrap_torch_tensor(indices), wrap_torch_tensor(inp)
    try:
        wgb.wholegraph_scatter_op(wn, wi, wg_table, env or wgb.cached_env_fns(), current_stream_int(), sms)
    finally:
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wn)
