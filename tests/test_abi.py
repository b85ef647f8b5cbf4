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


def test_every_wholegraph_function_has_a_wholememory_twin(wgb):
    """Binaries built against the older wholememory_* names of this C API find every function
    under that spelling too, at the same address."""
    lib = wgb.lib()
    names = [n for n in declared_functions() if n.startswith("wholegraph_") and not n.startswith("wholegraph_b200_")]
    assert "wholegraph_gather" in names and "wholegraph_scatter" in names
    for n in names:
        twin = "wholememory_" + n[len("wholegraph_"):]
        assert hasattr(lib, twin), f"{twin} is not exported"
        a = C.cast(getattr(lib, n), C.c_void_p).value
        b = C.cast(getattr(lib, twin), C.c_void_p).value
        assert a == b, f"{twin} is not {n}"


def test_wholememory_header_compiles_and_links(wgb, tmp_path):
    """A caller written against the wholememory_* spelling (types, enumerators, functions) builds
    with the alias header and runs against the library; no device is touched."""
    import shutil
    import subprocess
    cxx = shutil.which("g++")
    cuda_inc = "/usr/local/cuda/include"
    if cxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("needs g++ and the CUDA headers")
    src = tmp_path / "caller.cpp"
    src.write_text('''
#include <wholememory/wholememory.h>
#include <cstdio>
int main() {
  wholememory_tensor_description_t d;
  wholememory_initialize_tensor_desc(&d);
  d.dim = 1, d.sizes[0] = 7, d.dtype = WHOLEMEMORY_DT_INT64;
  if (!wholememory_unsqueeze_tensor(&d, 1) || d.dim != 2) return 2;
  if (wholememory_dtype_get_element_size(WHOLEMEMORY_DT_BF16) != 2) return 3;
  if ((int)WHOLEMEMORY_MT_CONTINUOUS != 1 || (int)WHOLEMEMORY_MT_DISTRIBUTED != 2 || (int)WHOLEMEMORY_MT_CHUNKED != 3) return 4;
  wholememory_env_func_t* env = nullptr;
  if (wholememory_gather(nullptr, nullptr, nullptr, env, nullptr, -1) != WHOLEMEMORY_INVALID_INPUT) return 5;
  if (wholememory_scatter(nullptr, nullptr, nullptr, env, nullptr, -1) != WHOLEMEMORY_INVALID_INPUT) return 6;
  if (wholememory_embedding_gather_gradient_apply(nullptr, nullptr, nullptr, false, 0.f, env, 0) == WHOLEMEMORY_SUCCESS) return 7;
  std::puts("ok");
  return 0;
}
''')
    lib_dir = os.path.dirname(wgb.LIB_PATH)
    exe = tmp_path / "caller"
    subprocess.run([cxx, "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc, str(src), "-L", lib_dir,
                    "-lwholegraph", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0 and res.stdout.strip() == "ok", (res.returncode, res.stdout, res.stderr)


def _signatures(header_dir):
    """{function name: (return type, [parameter types])} of the C declarations under a header
    directory, with comments, parameter names and default arguments taken out."""
    sigs = {}
    for path in glob.glob(os.path.join(header_dir, "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        text = re.sub(r"#[^\n]*(\\\n[^\n]*)*", "", text)
        text = re.sub(r"typedef[^;{]*\([^;]*;", "", text)             # function-pointer typedefs
        for m in re.finditer(r"([A-Za-z_][\w\s\*]*?[\s\*])((?:wholegraph_|get_|fork_|graph_|csr_|generate_)\w+)\s*\(([^;{]*?)\)\s*;", text):
            ret, name, params = m.group(1), m.group(2), m.group(3)
            ret = " ".join(ret.replace("extern", "").split())
            types = []
            for p in [x.strip() for x in params.split(",") if x.strip() and x.strip() != "void"]:
                p = p.split("=")[0].strip()
                p = re.sub(r"\b[A-Za-z_]\w*$", "", p).strip() if re.search(r"[\s\*&][A-Za-z_]\w*$", p) else p
                types.append(p.replace(" *", "*").replace("* ", "*").replace("  ", " "))
            sigs[name] = (ret.replace(" *", "*"), types)
    return sigs


def test_declarations_match_the_reference_headers():
    """When a checkout of the reference lies beside this repository (or WHOLEGRAPH_REFERENCE_CHECKOUT names
    one), every function its public headers declare is declared here with the same return type and
    the same parameter types, in order."""
    ref = os.environ.get("WHOLEGRAPH_REFERENCE_CHECKOUT") or os.path.join(os.path.dirname(ROOT), "reference")
    ref_dir = os.path.join(ref, "cpp", "include", "wholegraph")
    if not os.path.isdir(ref_dir):
        pytest.skip("no reference checkout here")
    theirs, ours = _signatures(ref_dir), _signatures(os.path.join(ROOT, "include", "wholegraph"))
    assert len(theirs) >= 95, f"only {len(theirs)} declarations parsed from the reference headers"
    missing = sorted(set(theirs) - set(ours))
    assert not missing, f"declared by the reference, not here: {missing}"
    different = {n: (theirs[n], ours[n]) for n in theirs if theirs[n] != ours[n]}
    assert not different, f"signatures differ: {different}"
