"""GPU tests of wholegraph_load_from_file / wholegraph_store_to_file through the C ABI: dense rows in
one or several files into a (possibly wider) table and back, as the reference's loader does
(cpp/src/wholegraph/file_io.cpp:1849-2165; tensor-level argument rule of the reference binding,
python/pylibwholegraph/src/pylibwholegraph/binding/tensor_binding.hpp:504-540).  Bytes must match."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm(gpu, wgb):
    c = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    yield c
    wgb.destroy_communicator(c)


def _read_rows(gpu, torch, t, rows, dim, dtype):
    out = torch.empty((rows, dim), dtype=dtype, device="cuda")
    gpu.gather(t, torch.arange(rows, device="cuda", dtype=torch.int64), out)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("mem", ["MtContinuous", "MtDistributed", "MtChunked"])
@pytest.mark.parametrize("round_robin", [0, 7])
def test_load_several_files_then_store(gpu, wgb, comm, tmp_path, mem, round_robin):
    import torch
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    rows, dim = 1000, 20
    data = np.random.default_rng(3).integers(-2**31, 2**31 - 1, size=(rows, dim), dtype=np.int64).astype(np.int32)
    cuts = [0, 123, 124, 700, rows]                       # four files, one of a single record
    files = []
    for k in range(len(cuts) - 1):
        path = str(tmp_path / f"part_{k}.bin")
        data[cuts[k]:cuts[k + 1]].tofile(path)
        files.append(path)
    t = wgb.create_wholegraph_tensor(wgb.make_description([rows, dim], DT.DtInt), comm, getattr(MT, mem), ML.MlDevice)
    wgb.tensor_from_filelist(t, files, round_robin)     # one rank: round robin deals every block to rank 0
    assert np.array_equal(_read_rows(gpu, torch, t, rows, dim, torch.int32), data)
    out = str(tmp_path / "stored.bin")
    wgb.tensor_to_file(t, out)
    assert np.array_equal(np.fromfile(out, dtype=np.int32).reshape(rows, dim), data)
    wgb.destroy_wholegraph_tensor(t)


def test_load_into_a_column_view_of_a_wider_table(gpu, wgb, comm, tmp_path):
    """Records narrower than the table row, placed at a column offset: the rest of every row stays."""
    import torch
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    rows, stride, dim, col = 257, 24, 10, 8
    t = wgb.create_wholegraph_tensor(wgb.make_description([rows, stride], DT.DtFloat), comm, MT.MtContinuous,
                                     ML.MlDevice)
    base = torch.full((rows, stride), -1.0, device="cuda")
    gpu.scatter(base, torch.arange(rows, device="cuda", dtype=torch.int64), t)
    torch.cuda.synchronize()
    starts = (wgb.C.c_int64 * 2)(0, col)
    ends = (wgb.C.c_int64 * 2)(rows, col + dim)
    view = wgb.C.c_void_p()
    wgb.check(wgb.lib().wholegraph_tensor_get_subtensor(t, starts, ends, wgb.C.byref(view)), "subtensor")
    data = np.random.default_rng(4).uniform(-1, 1, size=(rows, dim)).astype(np.float32)
    path = str(tmp_path / "narrow.bin")
    data.tofile(path)
    wgb.tensor_from_filelist(view, [path])
    want = np.full((rows, stride), -1.0, dtype=np.float32)
    want[:, col:col + dim] = data
    assert np.array_equal(_read_rows(gpu, torch, t, rows, stride, torch.float32), want)
    out = str(tmp_path / "narrow_out.bin")
    wgb.tensor_to_file(view, out)
    assert np.array_equal(np.fromfile(out, dtype=np.float32).reshape(rows, dim), data)
    wgb.destroy_wholegraph_tensor(view)
    wgb.destroy_wholegraph_tensor(t)


def test_bad_files_are_refused(gpu, wgb, comm, tmp_path):
    MT, ML, DT = wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphDataType
    t = wgb.create_wholegraph_tensor(wgb.make_description([10, 4], DT.DtFloat), comm, MT.MtContinuous, ML.MlDevice)
    partial = str(tmp_path / "partial.bin")
    np.zeros(7, dtype=np.float32).tofile(partial)          # 28 bytes: not a multiple of a 16-byte record
    too_long = str(tmp_path / "long.bin")
    np.zeros((11, 4), dtype=np.float32).tofile(too_long)
    for files in ([partial], [str(tmp_path / "missing.bin")], [too_long]):
        with pytest.raises(wgb.WholeGraphError):
            wgb.tensor_from_filelist(t, files)
    wgb.destroy_wholegraph_tensor(t)
