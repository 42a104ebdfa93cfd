"""Regenerates tests/golden/weight_files/: a .nve container written by the UNMODIFIED reference
weight-file code (oracle/_ref/libnve_ref_ser.so, built from the reference checkout by
oracle/build.py) and, beside it, what the reference's numpy loader reads from two .npy files
(format versions 1.0 and 2.0) that numpy itself wrote.

    python tests/golden/make_weight_files.py
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
OUT = Path(__file__).resolve().parent / "weight_files"


def tensors():
    rng = np.random.default_rng(2024)
    return [(7, rng.normal(0, 1, (5, 8)).astype(np.float32)),
            (1 << 40, rng.normal(0, 1, (3, 16)).astype(np.float16)),
            (0, rng.integers(-100, 100, (4, 2)).astype(np.int64)),
            (12345, np.zeros((0, 4), np.float32))]


def load_reference():
    from oracle import build
    path = build.build_reference_serialization()
    if path is None:
        raise SystemExit("the reference checkout is not available: cannot regenerate the fixtures")
    lib = C.CDLL(str(path))
    lib.refser_last_error.restype = C.c_char_p
    return lib


def reference_write_nve(lib, path, items):
    n = len(items)
    names = (C.c_uint64 * n)(*[k for k, _ in items])
    data = (C.c_void_p * n)(*[a.ctypes.data if a.size else None for _, a in items])
    rows = (C.c_uint64 * n)(*[a.shape[0] for _, a in items])
    cols = (C.c_uint64 * n)(*[a.shape[1] for _, a in items])
    elem = (C.c_uint64 * n)(*[a.itemsize for _, a in items])
    if lib.refser_write_nve(str(path).encode(), n, names, data, rows, cols, elem) != 0:
        raise RuntimeError(lib.refser_last_error().decode())


def reference_numpy_rows(lib, path):
    rows, row_bytes = C.c_uint64(0), C.c_uint64(0)
    if lib.refser_numpy_info(str(path).encode(), C.byref(rows), C.byref(row_bytes)) != 0:
        raise RuntimeError(lib.refser_last_error().decode())
    out = np.zeros((rows.value, row_bytes.value), np.uint8)
    if lib.refser_numpy_load(str(path).encode(), rows.value, out.ctypes.data) != 0:
        raise RuntimeError(lib.refser_last_error().decode())
    return out


def main():
    lib = load_reference()
    OUT.mkdir(exist_ok=True)
    reference_write_nve(lib, OUT / "reference_written.nve", tensors())
    rng = np.random.default_rng(7)
    a = rng.normal(0, 1, (6, 3, 4)).astype(np.float32)          # rows of 12 elements
    np.save(OUT / "table_v1.npy", a)
    with open(OUT / "table_v2.npy", "wb") as f:
        np.lib.format.write_array(f, rng.integers(-5, 5, (9,)).astype(np.int64), version=(2, 0))
    np.savez(OUT / "reference_read.npz",
             table_v1=reference_numpy_rows(lib, OUT / "table_v1.npy"),
             table_v2=reference_numpy_rows(lib, OUT / "table_v2.npy"))
    print("wrote", sorted(p.name for p in OUT.iterdir()))


if __name__ == "__main__":
    main()
