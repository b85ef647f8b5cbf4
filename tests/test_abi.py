"""The shared library loads without a GPU and exports every function the public headers declare;
struct layouts and enum values match the reference ABI.  No compute call is made here."""
import ctypes as C
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DECL = re.compile(r"^\s*(?:[A-Za-z_][\w\s\*]*?[\s\*])?((?:wholegraph_|get_|fork_)\w+)\s*\(", re.M)


def declared_functions():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "wholegraph", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)          # comments
        text = re.sub(r"#define[^\n]*(\\\n[^\n]*)*", "", text)      # macros
        text = re.sub(r"typedef[^;]*;", "", text)                   # function-pointer typedefs
        for m in DECL.finditer(text):
            names.add(m.group(1))
    return sorted(names)


def test_headers_declare_the_expected_surface():
    names = declared_functions()
    for must in ("wholegraph_gather", "wholegraph_scatter", "wholegraph_embedding_gather_gradient_apply",
                 "wholegraph_malloc", "wholegraph_create_tensor", "wholegraph_create_communicator",
                 "wholegraph_b200_partition_by_owner", "fork_get_device_count", "get_wholegraph_tensor_count"):
        assert must in names
    assert len(names) > 90


def test_library_exports_every_declared_function(wgb):
    lib = wgb.lib()
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_struct_layouts_and_enums(wgb):
    assert C.sizeof(wgb.TensorDescription) == 8 * 8 * 2 + 8 + 4 + 4
    assert wgb.TensorDescription.storage_offset.offset == 128
    assert wgb.TensorDescription.dim.offset == 136 and wgb.TensorDescription.dtype.offset == 140
    assert C.sizeof(wgb.UniqueId) == 128
    assert C.sizeof(wgb.EnvFns) == 5 * 8 + 3 * 8
    lib = wgb.lib()
    sizes = {0: 0, 1: 4, 2: 2, 3: 8, 4: 2, 5: 4, 6: 8, 7: 2, 8: 1}     # wholegraph_dtype_t -> bytes
    for dt, sz in sizes.items():
        assert lib.wholegraph_dtype_get_element_size(dt) == sz
    assert [int(e) for e in wgb.ErrorCode] == list(range(11))
    assert int(wgb.WholeGraphMemoryType.MtContinuous) == 1 and int(wgb.WholeGraphMemoryType.MtDistributed) == 2
    assert int(wgb.WholeGraphOptimizerType.OptRmsProp) == 3 and int(wgb.WholeGraphOptimizerType.OptAdaGrad) == 4


def test_null_arguments_are_rejected_without_touching_a_device(wgb):
    lib = wgb.lib()
    bad = int(wgb.ErrorCode.INVALID_INPUT)
    assert lib.wholegraph_gather(None, None, None, None, None, -1) == bad
    assert lib.wholegraph_scatter(None, None, None, None, None, -1) == bad
    assert lib.wholegraph_malloc(None, 0, None, 1, 1, 1, None) == bad
    assert lib.wholegraph_create_tensor(None, None, None, 1, 1, None) == bad
    assert lib.wholegraph_communicator_barrier(None) == bad
    assert lib.wholegraph_embedding_gather(None, None, None, False, None, 0) == bad
    assert lib.wholegraph_b200_version().startswith(b"wholegraph-b200")


def test_loading_fails_loudly_without_the_library(wgb, tmp_path):
    with pytest.raises(RuntimeError, match="no CPU or Python fallback"):
        wgb.load_library(str(tmp_path / "libwholegraph.so"))
