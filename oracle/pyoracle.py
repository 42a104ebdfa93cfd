"""ctypes front-ends of the parity checker: the plain-C restatement (``libnve_oracle.so``) and the
unmodified reference CPU build (``libnve_ref.so``).  TEST INFRASTRUCTURE: only tests/, the smoke
entry and the benchmark's CPU-baseline legs may import this module.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build as _build

_vp, _i64, _i32 = C.c_void_p, C.c_int64, C.c_int

DT = {"f32": 1, "f16": 3, "qint8_f32": 7, "qint8_f16": 8, "quint8_f32": 9, "quint8_f16": 10}
NP_OF = {1: np.float32, 3: np.float16}
POOL = {"concat": 0, "sum": 1, "mean": 2, "wsum": 3, "wmean": 4}


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_vp)


class Oracle:
    """The C restatement."""

    def __init__(self):
        self.lib = C.CDLL(str(_build.build_oracle()))
        L = self.lib
        L.nve_oracle_gather.restype = _i64
        L.nve_oracle_gather.argtypes = [_vp, _i64, _i64, _vp, _i32, _i64, _vp, _i64, _vp]
        L.nve_oracle_lookup_pooled.restype = _i32
        L.nve_oracle_lookup_pooled.argtypes = [_vp, _i64, _i64, _i32, _i64, _i64, _vp, _i32, _i64,
                                               _i32, _i32, _vp, _i32, _i64, _i64, _vp, _i32, _vp,
                                               _i64, _i32]
        L.nve_oracle_update.restype = None
        L.nve_oracle_update.argtypes = [_vp, _i64, _i64, _vp, _i32, _i64, _vp, _i64]
        L.nve_oracle_update_accumulate.restype = _i32
        L.nve_oracle_update_accumulate.argtypes = [_vp, _i64, _i64, _i32, _vp, _i32, _i64, _vp, _i64]

    def gather(self, table2d: np.ndarray, keys: np.ndarray, out: np.ndarray, hit_mask=None) -> int:
        rows = table2d.reshape(table2d.shape[0], -1).view(np.uint8)
        return self.lib.nve_oracle_gather(_ptr(rows), rows.shape[0], rows.shape[1], _ptr(keys),
                                          keys.dtype.itemsize, keys.size, _ptr(out),
                                          out.strides[0], _ptr(hit_mask))

    def lookup_pooled(self, table_bytes: np.ndarray, value_dtype: str, row_width: int,
                      keys: np.ndarray, pooling: str, *, offsets=None, hotness=0, weights=None,
                      out_dtype: str = "f32", default_row: int = -1) -> np.ndarray:
        """table_bytes: [num_rows, row_stride] uint8 view of the stored rows."""
        assert table_bytes.dtype == np.uint8 and table_bytes.ndim == 2
        n = keys.size
        if pooling == "concat":
            num_bags = n
        elif offsets is not None:
            num_bags = offsets.size - 1
        else:
            num_bags = n // hotness
        out = np.zeros((num_bags, row_width), dtype=NP_OF[DT[out_dtype]])
        wdt = 0
        if weights is not None:
            wdt = DT["f32"] if weights.dtype == np.float32 else DT["f16"]
        rc = self.lib.nve_oracle_lookup_pooled(
            _ptr(table_bytes), table_bytes.shape[0], table_bytes.shape[1], DT[value_dtype],
            row_width, default_row, _ptr(keys), keys.dtype.itemsize, n, POOL[pooling],
            1 if offsets is not None else 0, _ptr(offsets),
            offsets.dtype.itemsize if offsets is not None else 8, num_bags, hotness,
            _ptr(weights), wdt, _ptr(out), out.strides[0] if num_bags else row_width * out.itemsize,
            DT[out_dtype])
        if rc != 0:
            raise ValueError("oracle: unsupported dtype combination")
        return out

    def update(self, table_bytes, keys, values_bytes):
        self.lib.nve_oracle_update(_ptr(table_bytes), table_bytes.shape[0], table_bytes.shape[1],
                                   _ptr(keys), keys.dtype.itemsize, keys.size, _ptr(values_bytes),
                                   values_bytes.strides[0])

    def update_accumulate(self, table: np.ndarray, keys, updates: np.ndarray):
        dt = DT["f32"] if table.dtype == np.float32 else DT["f16"]
        rc = self.lib.nve_oracle_update_accumulate(_ptr(table), table.shape[0], table.strides[0],
                                                   dt, _ptr(keys), keys.dtype.itemsize, keys.size,
                                                   _ptr(updates), updates.strides[0])
        assert rc == 0


class Reference:
    """The unmodified reference CPU path (HostEmbeddingLayer over a LinearHostTable)."""

    def __init__(self):
        path = _build.build_reference()
        if path is None or not Path(path).exists():
            raise FileNotFoundError("oracle/_ref/libnve_ref.so is not built and the reference "
                                    "checkout is absent")
        self.lib = C.CDLL(str(path))
        L = self.lib
        L.nve_ref_last_error.restype = C.c_char_p
        L.nve_ref_host_layer_create.restype = _vp
        L.nve_ref_host_layer_create.argtypes = [_vp, _i64, _i64, _i32]
        L.nve_ref_host_layer_destroy.argtypes = [_vp]
        L.nve_ref_num_workers.restype = _i64
        L.nve_ref_num_workers.argtypes = [_vp]
        L.nve_ref_host_layer_lookup.argtypes = [_vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _vp,
                                                _i64, _i64, _vp, _i32, _i32, _vp]
        L.nve_ref_host_layer_update.argtypes = [_vp, _i64, _vp, _i64, _i64, _vp]
        L.nve_ref_host_layer_accumulate.argtypes = [_vp, _i64, _vp, _i64, _i64, _vp, _i32]
        L.nve_ref_pool_gathered_i32.argtypes = [_vp, _i32, _i32, _i32, _i64, _i64, _vp, _i64, _vp,
                                                _i64, _i32, _i64, _vp, _i32, _vp]

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError("reference: " + (self.lib.nve_ref_last_error() or b"").decode())

    def layer(self, table_bytes: np.ndarray, value_dtype: str):
        return RefLayer(self, table_bytes, value_dtype)


class RefLayer:
    def __init__(self, ref: Reference, table_bytes: np.ndarray, value_dtype: str):
        assert table_bytes.dtype == np.uint8 and table_bytes.ndim == 2 and table_bytes.flags.c_contiguous
        self.ref, self.table, self.value_dtype = ref, table_bytes, value_dtype
        self.h = ref.lib.nve_ref_host_layer_create(_ptr(table_bytes), table_bytes.shape[0],
                                                   table_bytes.shape[1], DT[value_dtype])
        if not self.h:
            raise RuntimeError("reference: " + ref.lib.nve_ref_last_error().decode())

    @property
    def num_workers(self) -> int:
        return self.ref.lib.nve_ref_num_workers(self.h)

    def close(self):
        if self.h:
            self.ref.lib.nve_ref_host_layer_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def lookup(self, keys: np.ndarray, out: np.ndarray) -> float:
        hr = C.c_float(0)
        self.ref._check(self.ref.lib.nve_ref_host_layer_lookup(
            self.h, keys.size, _ptr(keys), _ptr(out), out.strides[0], 0, 0, 0, None, 0, 0, None, 0,
            0, C.byref(hr)))
        return hr.value

    def lookup_pooled(self, keys: np.ndarray, pooling: str, row_width: int, *, offsets=None,
                      hotness=0, weights=None, out_dtype="f32", out=None) -> np.ndarray:
        n = keys.size
        if pooling == "concat":
            num_bags = n
        elif offsets is not None:
            num_bags = offsets.size - 1
        else:
            num_bags = n // hotness
        if out is None:
            out = np.zeros((num_bags, row_width), dtype=NP_OF[DT[out_dtype]])
        wdt = 0
        if weights is not None:
            wdt = DT["f32"] if weights.dtype == np.float32 else DT["f16"]
        hr = C.c_float(0)
        self.ref._check(self.ref.lib.nve_ref_host_layer_lookup(
            self.h, n, _ptr(keys), _ptr(out), out.strides[0], 1, POOL[pooling],
            1 if offsets is not None else 0, _ptr(offsets),
            offsets.size if offsets is not None else 0, hotness, _ptr(weights), wdt,
            DT[out_dtype], C.byref(hr)))
        return out

    def update(self, keys, values_bytes):
        self.ref._check(self.ref.lib.nve_ref_host_layer_update(
            self.h, keys.size, _ptr(keys), values_bytes.strides[0], values_bytes.shape[1],
            _ptr(values_bytes)))

    def accumulate(self, keys, updates: np.ndarray):
        self.ref._check(self.ref.lib.nve_ref_host_layer_accumulate(
            self.h, keys.size, _ptr(keys), updates.strides[0],
            updates.shape[1] * updates.itemsize, _ptr(updates), DT["f32"]))

    def pool_gathered_i32(self, gathered_bytes: np.ndarray, row_width: int, pooling: str,
                          offsets32: np.ndarray, weights=None, out_dtype="f32") -> np.ndarray:
        num_bags = offsets32.size - 1
        out = np.zeros((num_bags, row_width), dtype=NP_OF[DT[out_dtype]])
        wdt = 0
        if weights is not None:
            wdt = DT["f32"] if weights.dtype == np.float32 else DT["f16"]
        self.ref._check(self.ref.lib.nve_ref_pool_gathered_i32(
            self.h, DT[self.value_dtype], DT[out_dtype], wdt, num_bags, row_width,
            _ptr(gathered_bytes), gathered_bytes.strides[0], _ptr(out), out.strides[0], 1, 0,
            _ptr(offsets32), POOL[pooling], _ptr(weights)))
        return out
