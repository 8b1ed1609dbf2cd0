"""Raw tensor files and perf.txt in the reference harness's formats (CPU only: no kernel runs)."""
import re
import struct

import numpy as np
import pytest


def reference_reader(path):
    """What the reference's host does with an output file (backend/hexagon_executor.py:200-216)."""
    ids = {0: np.bool_, 1: np.float16, 2: np.float32, 3: np.float64, 4: np.int8, 5: np.int16, 6: np.int32,
           7: np.int64, 8: np.uint8, 9: np.uint16, 10: np.uint32}  # test/utils/dsp/include/tensor.h:26-38
    with open(path, "rb") as f:
        dtype_id = struct.unpack("I", f.read(4))[0]
        rank = struct.unpack("q", f.read(8))[0]
        shape = [struct.unpack("q", f.read(8))[0] for _ in range(rank)]
        data = f.read()
    return np.frombuffer(data, dtype=ids[dtype_id]).reshape(shape)


@pytest.mark.parametrize("dtype,shape", [(np.float16, (5, 7)), (np.float32, (3,)), (np.int8, (2, 3, 4)),
                                         (np.int32, (4, 4)), (np.float16, ()), (np.uint8, (0, 8)),
                                         (np.int64, (2, 2)), (np.float64, (1, 9))])
def test_dump_is_what_the_reference_reader_expects(hm, tmp_path, dtype, shape):
    rng = np.random.Generator(np.random.Philox(7))
    t = (rng.normal(0, 10, shape) if np.dtype(dtype).kind == "f" else rng.integers(0, 100, shape)).astype(dtype)
    p = tmp_path / "out.bin"
    hm.tensor_dump(p, t)
    got = reference_reader(p)
    assert got.dtype == np.dtype(dtype) and got.shape == tuple(shape)
    assert got.tobytes() == t.tobytes()
    assert p.stat().st_size == 4 + 8 + 8 * len(shape) + t.nbytes
    dt, shp = hm.tensor_file_info(p)
    assert dt == np.dtype(dtype) and shp == tuple(shape)
    back = hm.tensor_load(p)
    assert back.dtype == t.dtype and np.array_equal(back, t)


def test_input_files_are_raw_data(hm, tmp_path):
    """Inputs carry no header (tensor.h:219-234): the caller's tensor supplies shape and type."""
    t = np.arange(24, dtype=np.float16).reshape(4, 6)
    p = tmp_path / "in.bin"
    p.write_bytes(t.tobytes())
    out = np.zeros((4, 6), np.float16)
    hm.tensor_load(p, out=out, has_header=False)
    assert np.array_equal(out, t)
    with pytest.raises(hm.B200Error):  # asks for more than the file holds
        hm.tensor_load(p, out=np.zeros((5, 6), np.float16), has_header=False)


def test_malformed_files_are_refused(hm, tmp_path):
    p = tmp_path / "bad.bin"
    p.write_bytes(struct.pack("<Iq", 1, 2) + struct.pack("<qq", 4, 4) + b"\0" * 10)  # 32 bytes of data needed
    with pytest.raises(hm.B200Error):
        hm.tensor_file_info(p)
    p.write_bytes(struct.pack("<Iq", 42, 1) + struct.pack("<q", 1) + b"\0")  # unknown dtype id
    with pytest.raises(hm.B200Error):
        hm.tensor_file_info(p)
    p.write_bytes(b"\1\0")  # truncated header
    with pytest.raises(hm.B200Error):
        hm.tensor_load(p)
    with pytest.raises(hm.B200Error):
        hm.tensor_file_info(tmp_path / "missing.bin")


def test_perf_report_text(hm, tmp_path):
    """Byte-for-byte what TestReport::save + the appended cycle line produce
    (test_report.h:43-50, hexagon_launcher_base.py:189-192)."""
    p = tmp_path / "perf.txt"
    hm.perf_report_save(p, "matmul", 52.25, "us", "Pass", cycles=112345)
    text = p.read_text()
    assert text == "Test_Info: {\n\tName:matmul\n\tResult:Pass\n\tPerf:52.250000\n\tUnits:us\n}\nPerfPcycles:112345\n"
    # the reference's parsers: first line containing "Result" (hexagon_executor.py:102-106),
    # the cycle line (hmx_search.py:1075)
    first = next(line for line in text.splitlines() if "Result" in line)
    assert first.split("Result:")[-1].strip() == "Pass"
    assert re.search(r"^PerfPcycles:\s*([0-9]+)", text, re.MULTILINE).group(1) == "112345"
    hm.perf_report_save(p, "softmax_kernel", 3.0, "us", "Fail")
    assert p.read_text() == "Test_Info: {\n\tName:softmax_kernel\n\tResult:Fail\n\tPerf:3.000000\n\tUnits:us\n}\n"
    hm.perf_report_save(p, "x", 0.0, "microseconds", "???")
    assert "Result:Unknown" in p.read_text()


def test_manifest_starts_empty(hm):
    hm.manifest_reset()
    assert hm.manifest() == {"matmuls": []}
