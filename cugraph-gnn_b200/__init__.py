"""wholegraph-b200: the WholeGraph embedding gather / scatter / sparse-optimizer hot path as
hand-written sm_100a kernels behind the reference's C ABI.

`binding` is the ctypes mirror of the C headers in include/wholegraph/; `torch_utils` wraps
torch tensors for it; `build.build()` compiles libwholegraph.so in place.
"""
from . import binding  # noqa: F401
from .build import build  # noqa: F401

__all__ = ["binding", "build"]
