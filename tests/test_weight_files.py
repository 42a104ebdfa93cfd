"""Weight-file formats (weight_files.py) against files written and read by the UNMODIFIED reference
code: committed fixtures (tests/golden/weight_files, made by make_weight_files.py) and, where the
compiled reference is at hand, live round trips in both directions."""
import ctypes as C
import io
import sys
from pathlib import Path

import numpy as np
import pytest

from nv_embedding_cache_b200 import weight_files as wf

GOLD = Path(__file__).resolve().parent / "golden" / "weight_files"
sys.path.insert(0, str(GOLD.parent))
from make_weight_files import tensors  # noqa: E402


def test_reader_reads_the_reference_written_container():
    with open(GOLD / "reference_written.nve", "rb") as f:
        assert wf.verify_header(f)
        listed = wf.list_tensors(f)
        assert listed == [(k, a.shape[0], a.shape[1], a.itemsize) for k, a in tensors()]
        for name, want in reversed(tensors()):            # any order: the reader walks the entries
            got = np.full_like(want, 1)
            assert wf.read_tensor(f, name, got)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
        assert not wf.read_tensor(f, 999, np.zeros((1, 1), np.float32))
        with pytest.raises(ValueError):
            wf.read_tensor(f, 7, np.zeros((5, 9), np.float32))     # stored size differs


def test_writer_is_byte_identical_to_the_reference_writer():
    buf = io.BytesIO()
    wf.write_header(buf)
    for name, a in tensors():
        wf.write_tensor(buf, name, a)
    assert buf.getvalue() == (GOLD / "reference_written.nve").read_bytes()
    with pytest.raises(ValueError):
        wf.write_tensor(buf, 1, np.zeros((2, 1 << 16), np.uint8))


def test_bad_container_header():
    assert not wf.verify_header(io.BytesIO(b"\x00" * 12))
    assert not wf.verify_header(io.BytesIO(b"\x00\x45\x56\x4e"))
    with pytest.raises(ValueError):
        wf.read_tensor(io.BytesIO(b"NVE?" + b"\x00" * 8), 0, np.zeros((1, 1), np.float32))


@pytest.mark.parametrize("name", ["table_v1", "table_v2"])
def test_numpy_table_reads_what_the_reference_reads(name):
    want = np.load(GOLD / "reference_read.npz")[name]
    with open(GOLD / f"{name}.npy", "rb") as f:
        t = wf.NumpyTable(f)
        assert (t.get_num_rows(), t.get_row_size_in_bytes()) == want.shape
        assert not t.fortran_order
        t.reset()
        first = want.shape[0] // 2
        got = np.concatenate([t.load_batch(first), t.load_batch(want.shape[0] - first)])
        assert np.array_equal(got, want)
        dest = np.zeros_like(want)
        assert wf.load_table(t, dest, batch_rows=4) == want.shape[0]
        assert np.array_equal(dest, want)
        with pytest.raises(ValueError):
            t.load_batch(1)                                  # past the end


def npy_bytes(a, version=(1, 0)):
    b = io.BytesIO()
    np.lib.format.write_array(b, a, version=version)
    return b.getvalue()


def test_numpy_table_refusals():
    ok = npy_bytes(np.zeros((4, 3), np.float32))
    assert wf.NumpyTable(io.BytesIO(ok)).get_shape() == [4, 3]
    assert wf.NumpyTable(io.BytesIO(npy_bytes(np.zeros(5, np.int32)))).get_row_size_in_bytes() == 4
    for bad in (b"\x93NUMPX" + ok[6:],                      # magic
                ok[:6] + b"\x03\x00" + ok[8:],              # version 3.0
                npy_bytes(np.zeros((2, 2), np.float16)),    # dtype outside the four
                ok[:-1],                                    # truncated data
                ok.replace(b"(4, 3)", b"(-4, 3"[:6])):      # unparsable shape
        with pytest.raises(ValueError):
            wf.NumpyTable(io.BytesIO(bad))


def test_binary_table():
    rows = np.arange(7 * 10, dtype=np.uint8).reshape(7, 10)
    t = wf.BinaryTable(io.BytesIO(rows.tobytes() + b"xyz"), 10)     # a trailing partial row is ignored
    assert t.get_num_rows() == 7
    dest = np.zeros((7, 10), np.uint8)
    assert wf.load_table(t, dest, batch_rows=3) == 7
    assert np.array_equal(dest, rows)


def test_live_round_trips_with_the_compiled_reference(tmp_path):
    from oracle import build
    path = build.build_reference_serialization()
    if path is None:
        pytest.skip("the compiled reference weight-file code is not available")
    lib = C.CDLL(str(path))
    rng = np.random.default_rng(11)
    items = [(3, rng.normal(0, 1, (33, 7)).astype(np.float32)), (2**63 + 5, rng.integers(0, 255, (2, 100)).astype(np.uint8))]
    mine = tmp_path / "mine.nve"
    with open(mine, "wb+") as f:
        wf.write_header(f)
        for name, a in items:
            wf.write_tensor(f, name, a)
    for name, a in items:                                    # the reference reads this library's file
        out = np.zeros_like(a)
        assert lib.refser_read_nve(str(mine).encode(), C.c_uint64(name), a.shape[0], a.shape[1], a.itemsize,
                                   out.ctypes.data) == 0
        assert np.array_equal(out, a)
    npy = tmp_path / "t.npy"
    a = rng.normal(0, 1, (50, 6)).astype(np.float64)
    np.save(npy, a)
    rows, rb = C.c_uint64(0), C.c_uint64(0)
    assert lib.refser_numpy_info(str(npy).encode(), C.byref(rows), C.byref(rb)) == 0
    with open(npy, "rb") as f:
        t = wf.NumpyTable(f)
        assert (t.get_num_rows(), t.get_row_size_in_bytes()) == (rows.value, rb.value)
    raw = tmp_path / "t.bin"
    raw.write_bytes(a.tobytes() + b"12345")
    n = C.c_uint64(0)
    assert lib.refser_binary_load(str(raw).encode(), 48, C.byref(n), None, 0) == 0
    with open(raw, "rb") as f:
        assert wf.BinaryTable(f, 48).get_num_rows() == n.value == 50
