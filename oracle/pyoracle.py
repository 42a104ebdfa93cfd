"""ctypes front-ends of the parity checker: the plain-C restatement (``libnve_oracle.so``), the
unmodified reference CPU build (``libnve_ref.so``) and the unmodified reference GPU code
(``libnve_ref_gpu.so``).  TEST INFRASTRUCTURE: only tests/, the smoke
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

    def dedup(self, keys: np.ndarray, max_run: int = -1, end_bit: int = 0):
        """Returns dict(unique, counts, inverse, offsets, loc_map, num_unique, num_chunks)."""
        L = self.lib
        L.nve_oracle_dedup.restype = None
        L.nve_oracle_dedup.argtypes = [_vp, _i32, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp]
        n = keys.size
        cap = n + (n // max_run if max_run > 0 else 0) + 2
        unique = np.zeros(n + 1, np.int64)
        counts = np.zeros(n + 1, np.int64)
        inverse = np.zeros(n + 1, np.int64)
        offsets = np.zeros(cap + 1, np.int64)
        loc_map = np.zeros(cap + 1, np.int64)
        runs = np.zeros(2, np.int64)
        L.nve_oracle_dedup(_ptr(keys), keys.dtype.itemsize, n, max_run, end_bit, _ptr(unique),
                           _ptr(counts), _ptr(inverse), _ptr(offsets), _ptr(loc_map), _ptr(runs))
        u, c = int(runs[0]), int(runs[1])
        return dict(unique=unique[:u], counts=counts[:u], inverse=inverse[:n], offsets=offsets[:c + 1],
                    loc_map=loc_map[:c] if max_run > 0 else None, num_unique=u, num_chunks=c)

    def dedup_grads(self, grads: np.ndarray, d: dict) -> np.ndarray:
        L = self.lib
        L.nve_oracle_dedup_grads.restype = None
        L.nve_oracle_dedup_grads.argtypes = [_vp, _i64, _i64, _vp, _vp, _vp, _i64, _vp, _i64]
        out = np.zeros((d["num_unique"], grads.shape[1]), np.float32)
        L.nve_oracle_dedup_grads(_ptr(grads), grads.strides[0] // 4, grads.shape[1],
                                 _ptr(d["inverse"]), _ptr(d["offsets"]), _ptr(d["loc_map"]),
                                 d["num_chunks"], _ptr(out), grads.shape[1])
        return out

    def pooling_backprop(self, keys: np.ndarray, csr: np.ndarray, bag_grads: np.ndarray, pooling: str,
                         weights: np.ndarray | None = None, max_run: int = 1024):
        """Backward of a pooled lookup: (unique keys, per-key gradient sums).  Per position the
        gradient is fl32(w * bag_grad[bag]) with w = 1, 1/len, weight or weight / sum of the bag's
        weights (fp32 sum in bag order, IEEE division); positions of a key are then added in the
        order of dedup_grads (cuda_ops/gradient_calculator.cuh:85-136,254-286)."""
        n = keys.size
        lens = np.diff(csr)
        bag = np.repeat(np.arange(lens.size), lens)
        w = np.ones(n, np.float32) if weights is None or pooling in ("sum", "mean") else weights.astype(np.float32)
        if pooling in ("mean", "wmean"):
            sums = np.zeros(lens.size, np.float32)
            for b in range(lens.size):          # fp32, in bag order
                acc = np.float32(0)
                for i in range(csr[b], csr[b + 1]):
                    acc = np.float32(acc + w[i])
                sums[b] = acc
            w = (w / sums[bag]).astype(np.float32)
        per_pos = (w[:, None] * bag_grads.astype(np.float32)[bag]).astype(np.float32)
        d = self.dedup(keys, max_run=max_run)
        return d["unique"], self.dedup_grads(per_pos, d)

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


class OracleCache:
    """The C restatement of the set-associative cache with the device-side modify policy."""

    def __init__(self, oracle: Oracle, cache_bytes: int, row_bytes: int, key_dtype=np.int64,
                 decay_rate: float = 0.95, sentinel: int = -1):
        L = self.lib = oracle.lib
        u64 = C.c_uint64
        L.nve_oracle_cache_num_sets.restype = u64
        L.nve_oracle_cache_num_sets.argtypes = [u64, _i64, _i32]
        L.nve_oracle_cache_create.restype = _vp
        L.nve_oracle_cache_create.argtypes = [u64, _i64, _i32, C.c_float, _i64]
        L.nve_oracle_cache_destroy.argtypes = [_vp]
        L.nve_oracle_cache_sets.restype = u64
        L.nve_oracle_cache_sets.argtypes = [_vp]
        for name in ("get_tags", "get_counters", "get_data"):
            getattr(L, "nve_oracle_cache_" + name).argtypes = [_vp, _vp]
        L.nve_oracle_cache_misses.restype = _i64
        L.nve_oracle_cache_misses.argtypes = [_vp]
        L.nve_oracle_cache_reset_misses.argtypes = [_vp]
        L.nve_oracle_cache_lookup.restype = _i64
        L.nve_oracle_cache_lookup.argtypes = [_vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _vp, _vp]
        L.nve_oracle_cache_insert.restype = _i64
        L.nve_oracle_cache_insert.argtypes = [_vp, _vp, _i64, _vp, _i64, _i32, _i64]
        L.nve_oracle_cache_update.argtypes = [_vp, _vp, _i64, _vp, _i64]
        L.nve_oracle_cache_update_accumulate.argtypes = [_vp, _vp, _i64, _vp, _i64, _i32]
        L.nve_oracle_cache_invalidate.argtypes = [_vp, _vp, _i64]
        L.nve_oracle_cache_clear.argtypes = [_vp]
        self.key_dtype = np.dtype(key_dtype)
        self.row_bytes = row_bytes
        self.h = L.nve_oracle_cache_create(cache_bytes, row_bytes, self.key_dtype.itemsize,
                                           decay_rate, sentinel)
        if not self.h:
            raise ValueError("cache too small for one set")
        self.num_sets = int(L.nve_oracle_cache_sets(self.h))
        self.sentinel = sentinel

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.nve_oracle_cache_destroy(self.h)
            self.h = None

    def _keys(self, keys):
        return np.ascontiguousarray(keys, dtype=self.key_dtype)

    def tags(self) -> np.ndarray:
        out = np.zeros((self.num_sets, 8), dtype=np.int64)
        self.lib.nve_oracle_cache_get_tags(self.h, _ptr(out))
        return out

    def counters(self) -> np.ndarray:
        out = np.zeros((self.num_sets, 8), dtype=np.float32)
        self.lib.nve_oracle_cache_get_counters(self.h, _ptr(out))
        return out

    def data(self) -> np.ndarray:
        out = np.zeros((self.num_sets, 8, self.row_bytes), dtype=np.uint8)
        self.lib.nve_oracle_cache_get_data(self.h, _ptr(out))
        return out

    def resident_keys(self) -> np.ndarray:
        """Keys held by the cache, in (set, way) order (get_keys_stored_in_cache)."""
        t = self.tags()
        sets = np.repeat(np.arange(self.num_sets, dtype=np.uint64), 8).reshape(t.shape)
        valid = t != self.sentinel
        if self.key_dtype.itemsize == 4:
            keys = (t.astype(np.uint32).astype(np.uint64) * np.uint64(self.num_sets) + sets).astype(np.uint32).view(np.int32)
        else:
            keys = (t.view(np.uint64) * np.uint64(self.num_sets) + sets).view(np.int64)
        return keys[valid]

    @property
    def misses(self) -> int:
        return int(self.lib.nve_oracle_cache_misses(self.h))

    def reset_misses(self):
        self.lib.nve_oracle_cache_reset_misses(self.h)

    def lookup(self, keys, out=None, hit_mask=None, table=None, default_row=-1, want_miss_list=False):
        keys = self._keys(keys)
        n = keys.size
        mp = np.zeros(n, dtype=np.int64) if want_miss_list else None
        mk = np.zeros(n, dtype=np.int64) if want_miss_list else None
        trows = 0 if table is None else table.shape[0]
        unresolved = self.lib.nve_oracle_cache_lookup(
            self.h, _ptr(keys), n, _ptr(out), out.strides[0] if out is not None else 0,
            _ptr(hit_mask), _ptr(table), trows, default_row, _ptr(mp), _ptr(mk))
        if want_miss_list:
            return unresolved, mp[:unresolved], mk[:unresolved]
        return unresolved

    def insert(self, keys, values=None, table=None, max_modify=1 << 20) -> int:
        keys = self._keys(keys)
        if table is not None:
            return self.lib.nve_oracle_cache_insert(self.h, _ptr(keys), keys.size, _ptr(table),
                                                    table.strides[0], 1, max_modify)
        return self.lib.nve_oracle_cache_insert(self.h, _ptr(keys), keys.size, _ptr(values),
                                                values.strides[0], 0, max_modify)

    def update(self, keys, values):
        keys = self._keys(keys)
        self.lib.nve_oracle_cache_update(self.h, _ptr(keys), keys.size, _ptr(values), values.strides[0])

    def update_accumulate(self, keys, updates):
        keys = self._keys(keys)
        self.lib.nve_oracle_cache_update_accumulate(self.h, _ptr(keys), keys.size, _ptr(updates),
                                                    updates.strides[0], int(updates.dtype == np.float16))

    def invalidate(self, keys):
        keys = self._keys(keys)
        self.lib.nve_oracle_cache_invalidate(self.h, _ptr(keys), keys.size)

    def clear(self):
        self.lib.nve_oracle_cache_clear(self.h)


class Reference:
    """The unmodified reference CPU path (HostEmbeddingLayer over a LinearHostTable)."""

    def __init__(self, for_timing: bool = False):
        """for_timing: take the AVX-512 build when this host has the instructions (what the
        reference's own build would pick here); parity checks always use the -mavx2 build."""
        path = None
        self.simd = "avx2"
        if for_timing and _build.host_has_avx512():
            path = _build.build_reference(avx512=True)
            if path is not None and Path(path).exists():
                self.simd = "avx512"
            else:
                path = None
        if path is None:
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


class ReferenceGpu:
    """The unmodified reference GPU code (``libnve_ref_gpu.so``): cache with device-side modify,
    Deduper, gradient de-duplication and the pooled find_and_combine kernel.  All pointers are raw
    device addresses (ints); every call synchronises the device before it returns."""

    def __init__(self):
        path = _build.build_reference_gpu()
        if path is None or not Path(path).exists():
            raise FileNotFoundError("libnve_ref_gpu.so is not built and the reference checkout is absent")
        self.lib = L = C.CDLL(str(path))
        f32 = C.c_float
        pp = C.POINTER(_vp)
        L.refgpu_last_error.restype = C.c_char_p
        sigs = {
            "refgpu_cache_create": [pp, _i64, _i64, _i64, f32, _i64],
            "refgpu_cache_destroy": [_vp],
            "refgpu_cache_view": [_vp, C.POINTER(_i64), pp, pp],
            "refgpu_cache_insert": [_vp, _vp, _i64, _vp, _i64],
            "refgpu_cache_insert_from_table": [_vp, _vp, _i64, _vp, _i64],
            "refgpu_cache_lookup_mask": [_vp, _vp, _i64, _vp, _i64, _vp, C.POINTER(_i64)],
            "refgpu_cache_lookup_table": [_vp, _vp, _i64, _vp, _i64, _vp, C.POINTER(_i64)],
            "refgpu_cache_find_and_combine": [_vp, _i64, _vp, pp, _i32, _i32, _i32, _vp, _i32, _i32,
                                              C.POINTER(C.c_float)],
            "refgpu_cache_lookup_table_timed": [_vp, pp, _i32, _i64, _vp, _i64, _vp, _i32, _i32,
                                                C.POINTER(f32)],
            "refgpu_cache_update": [_vp, _vp, _i64, _vp, _i64],
            "refgpu_cache_update_accumulate": [_vp, _vp, _i64, _vp, _i64, _i32],
            "refgpu_cache_invalidate": [_vp, _vp, _i64],
            "refgpu_cache_clear": [_vp],
            "refgpu_hostcache_create": [pp, _i64, _i64, _i64, f32, _i64],
            "refgpu_hostcache_destroy": [_vp],
            "refgpu_hostcache_view": [_vp, C.POINTER(_i64), pp, pp],
            "refgpu_hostcache_insert": [_vp, _vp, _i64, _vp, _i64, _i32],
            "refgpu_hostcache_update": [_vp, _vp, _i64, _vp, _i64],
            "refgpu_hostcache_update_accumulate": [_vp, _vp, _i64, _vp, _i64, _i32],
            "refgpu_hostcache_invalidate": [_vp, _vp, _i64],
            "refgpu_hostcache_clear": [_vp],
            "refgpu_hostcache_lookup_mask": [_vp, _vp, _i64, _vp, _i64, _vp],
            "refgpu_deduper_create": [pp, _i32, _i64],
            "refgpu_deduper_destroy": [_vp],
            "refgpu_deduper_dedup": [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i32],
            "refgpu_dedup_grads": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32],
            "refgpu_dedup_grads_f16": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32],
            "refgpu_dedup_grads_timed": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32,
                                         C.POINTER(f32)],
            "refgpu_update_accumulate_table": [_vp, _vp, _vp, _i32, _i64, _i64, _i32, _i32, C.POINTER(f32)],
            "refgpu_pooling_backprop": [_vp, _i64, _vp, _i64, _vp, _vp, _i32, _i32, _vp, _vp, C.POINTER(_i64)],
            "refgpu_find_and_combine": [_i32, _i64, _vp, pp, pp, _i32, _i32, _i32, _vp, _i32, _i32,
                                        C.POINTER(f32)],
        }
        for name, args in sigs.items():
            fn = getattr(L, name)
            fn.restype = _i32
            fn.argtypes = args

    def check(self, rc):
        if rc != 0:
            raise RuntimeError("reference GPU code: " + self.lib.refgpu_last_error().decode())

    # ---- cache
    def cache(self, cache_bytes, row_bytes, sentinel=-1, decay=0.95, max_modify=1 << 20):
        return RefGpuCache(self, cache_bytes, row_bytes, sentinel, decay, max_modify)

    def host_cache(self, cache_bytes, row_bytes, sentinel=-1, decay=0.95, max_modify=1 << 20):
        return RefGpuHostCache(self, cache_bytes, row_bytes, sentinel, decay, max_modify)

    def update_accumulate_table(self, src_ptr, keys_ptr, table_ptr, width, n, num_rows, warmup=0, iters=0):
        """table[keys[i]] += src[i] (fp32 rows); returns mean ms per call when iters > 0."""
        ms = C.c_float(0)
        self.check(self.lib.refgpu_update_accumulate_table(src_ptr, keys_ptr, table_ptr, width, n, num_rows,
                                                           warmup, iters, C.byref(ms)))
        return ms.value

    def pooling_backprop(self, keys_ptr, n, csr_ptr, num_bags, grads_ptr, weights_ptr, pooling, width,
                         unique_ptr, out_ptr) -> int:
        """pooling: "sum", "mean", "wsum", "wmean" (the mean forms need weights)."""
        u = _i64(0)
        self.check(self.lib.refgpu_pooling_backprop(keys_ptr, n, csr_ptr, num_bags, grads_ptr, weights_ptr,
                                                    POOL[pooling], width, unique_ptr, out_ptr, C.byref(u)))
        return u.value

    def deduper(self, max_run, max_keys):
        return RefGpuDeduper(self, max_run, max_keys)

    # ---- pooled lookup (kind: "f16_csr_mean", "f16_fixed_sum", "qint8_fixed_sum")
    KINDS = {"f16_csr_mean": 0, "f16_fixed_sum": 1, "qint8_fixed_sum": 2}

    def find_and_combine(self, kind, bags, table_ptr, key_ptrs, offset_ptrs, hot, width, out_ptr,
                         warmup=0, iters=0):
        nb = len(key_ptrs)
        keys = (_vp * nb)(*key_ptrs)
        offs = (_vp * nb)(*offset_ptrs) if offset_ptrs else None
        ms = C.c_float(0)
        self.check(self.lib.refgpu_find_and_combine(self.KINDS[kind], bags, table_ptr, keys, offs, nb,
                                                    hot, width, out_ptr, warmup, iters, C.byref(ms)))
        return ms.value


class RefGpuCache:
    def __init__(self, ref: ReferenceGpu, cache_bytes, row_bytes, sentinel, decay, max_modify):
        self.ref = ref
        self.h = _vp()
        ref.check(ref.lib.refgpu_cache_create(C.byref(self.h), cache_bytes, row_bytes, sentinel, decay,
                                              max_modify))
        self.row_bytes = row_bytes

    def close(self):
        if self.h:
            self.ref.check(self.ref.lib.refgpu_cache_destroy(self.h))
            self.h = _vp()

    def view(self):
        """(num_sets, device address of the tags [num_sets][8], device address of the rows)."""
        n, tags, rows = _i64(0), _vp(), _vp()
        self.ref.check(self.ref.lib.refgpu_cache_view(self.h, C.byref(n), C.byref(tags), C.byref(rows)))
        return n.value, tags.value, rows.value

    def insert(self, keys_ptr, n, values_ptr, stride):
        self.ref.check(self.ref.lib.refgpu_cache_insert(self.h, keys_ptr, n, values_ptr, stride))

    def insert_from_table(self, keys_ptr, n, table_ptr, stride):
        self.ref.check(self.ref.lib.refgpu_cache_insert_from_table(self.h, keys_ptr, n, table_ptr, stride))

    def lookup_mask(self, keys_ptr, n, out_ptr, stride, mask_ptr) -> int:
        m = _i64(0)
        self.ref.check(self.ref.lib.refgpu_cache_lookup_mask(self.h, keys_ptr, n, out_ptr, stride, mask_ptr,
                                                             C.byref(m)))
        return m.value

    def lookup_table(self, keys_ptr, n, out_ptr, stride, table_ptr) -> int:
        m = _i64(0)
        self.ref.check(self.ref.lib.refgpu_cache_lookup_table(self.h, keys_ptr, n, out_ptr, stride, table_ptr,
                                                              C.byref(m)))
        return m.value

    def find_and_combine(self, bags, table_ptr, key_ptrs, hot, width, out_ptr, warmup=0, iters=0) -> float:
        """The reference's pooled lookup with this cache in front of `table_ptr` (fp16 rows, fixed
        hotness, sum, fp16 out); mean milliseconds per launch when iters > 0."""
        nb = len(key_ptrs)
        ms = C.c_float(0)
        self.ref.check(self.ref.lib.refgpu_cache_find_and_combine(
            self.h, bags, table_ptr, (_vp * nb)(*key_ptrs), nb, hot, width, out_ptr, warmup, iters, C.byref(ms)))
        return ms.value

    def lookup_table_timed(self, key_ptrs, n, out_ptr, stride, table_ptr, warmup, iters) -> float:
        nb = len(key_ptrs)
        ms = C.c_float(0)
        self.ref.check(self.ref.lib.refgpu_cache_lookup_table_timed(
            self.h, (_vp * nb)(*key_ptrs), nb, n, out_ptr, stride, table_ptr, warmup, iters, C.byref(ms)))
        return ms.value

    def update(self, keys_ptr, n, values_ptr, stride):
        self.ref.check(self.ref.lib.refgpu_cache_update(self.h, keys_ptr, n, values_ptr, stride))

    def update_accumulate(self, keys_ptr, n, values_ptr, stride, fp16=False):
        self.ref.check(self.ref.lib.refgpu_cache_update_accumulate(self.h, keys_ptr, n, values_ptr, stride,
                                                                   1 if fp16 else 0))

    def invalidate(self, keys_ptr, n):
        self.ref.check(self.ref.lib.refgpu_cache_invalidate(self.h, keys_ptr, n))

    def clear(self):
        self.ref.check(self.ref.lib.refgpu_cache_clear(self.h))


class RefGpuHostCache:
    """The reference cache with its host-side modify policy (CacheSAHostModify<int64, int64>): keys of
    the modifying calls are HOST addresses, rows are device addresses."""

    def __init__(self, ref: ReferenceGpu, cache_bytes, row_bytes, sentinel, decay, max_modify):
        self.ref = ref
        self.h = _vp()
        ref.check(ref.lib.refgpu_hostcache_create(C.byref(self.h), cache_bytes, row_bytes, sentinel, decay,
                                                  max_modify))
        self.row_bytes = row_bytes

    def close(self):
        if self.h:
            self.ref.check(self.ref.lib.refgpu_hostcache_destroy(self.h))
            self.h = _vp()

    def view(self):
        n, tags, rows = _i64(0), _vp(), _vp()
        self.ref.check(self.ref.lib.refgpu_hostcache_view(self.h, C.byref(n), C.byref(tags), C.byref(rows)))
        return n.value, tags.value, rows.value

    def insert(self, host_keys_ptr, n, values_ptr, stride, linear=False):
        self.ref.check(self.ref.lib.refgpu_hostcache_insert(self.h, host_keys_ptr, n, values_ptr, stride,
                                                            1 if linear else 0))

    def update(self, host_keys_ptr, n, values_ptr, stride):
        self.ref.check(self.ref.lib.refgpu_hostcache_update(self.h, host_keys_ptr, n, values_ptr, stride))

    def update_accumulate(self, host_keys_ptr, n, values_ptr, stride, fp16=False):
        self.ref.check(self.ref.lib.refgpu_hostcache_update_accumulate(self.h, host_keys_ptr, n, values_ptr, stride,
                                                                       1 if fp16 else 0))

    def invalidate(self, host_keys_ptr, n):
        self.ref.check(self.ref.lib.refgpu_hostcache_invalidate(self.h, host_keys_ptr, n))

    def clear(self):
        self.ref.check(self.ref.lib.refgpu_hostcache_clear(self.h))

    def lookup_mask(self, keys_ptr, n, out_ptr, stride, mask_ptr):
        self.ref.check(self.ref.lib.refgpu_hostcache_lookup_mask(self.h, keys_ptr, n, out_ptr, stride, mask_ptr))


class RefGpuDeduper:
    """Reference Deduper<int64_t, MAX_RUN> (max_run in {-1, 8, 1024}) on device buffers."""

    def __init__(self, ref: ReferenceGpu, max_run: int, max_keys: int):
        self.ref = ref
        self.h = _vp()
        ref.check(ref.lib.refgpu_deduper_create(C.byref(self.h), max_run, max_keys))

    def close(self):
        if self.h:
            self.ref.check(self.ref.lib.refgpu_deduper_destroy(self.h))
            self.h = _vp()

    def dedup(self, keys_ptr, n, unique_ptr, counts_ptr, loc_map_ptr, inverse_ptr, offsets_ptr, end_bit=0):
        runs = np.zeros(2, np.int64)
        self.ref.check(self.ref.lib.refgpu_deduper_dedup(self.h, keys_ptr, n, unique_ptr, counts_ptr,
                                                         loc_map_ptr, runs.ctypes.data, inverse_ptr,
                                                         offsets_ptr, end_bit))
        return int(runs[0]), int(runs[1])

    def grads_f16(self, grads_ptr, out_ptr, unique_ptr, inverse_ptr, loc_map_ptr, offsets_ptr, num_unique,
                  num_chunks, width):
        runs = np.array([num_unique, num_chunks], np.int64)
        self.ref.check(self.ref.lib.refgpu_dedup_grads_f16(grads_ptr, out_ptr, unique_ptr, inverse_ptr,
                                                           loc_map_ptr, offsets_ptr, runs.ctypes.data, width))

    def grads(self, grads_ptr, out_ptr, unique_ptr, inverse_ptr, loc_map_ptr, offsets_ptr, num_unique,
              num_chunks, width, warmup=0, iters=0):
        runs = np.array([num_unique, num_chunks], np.int64)
        if iters <= 0:
            self.ref.check(self.ref.lib.refgpu_dedup_grads(grads_ptr, out_ptr, unique_ptr, inverse_ptr,
                                                           loc_map_ptr, offsets_ptr, runs.ctypes.data, width))
            return 0.0
        ms = C.c_float(0)
        self.ref.check(self.ref.lib.refgpu_dedup_grads_timed(grads_ptr, out_ptr, unique_ptr, inverse_ptr,
                                                             loc_map_ptr, offsets_ptr, runs.ctypes.data,
                                                             width, warmup, iters, C.byref(ms)))
        return ms.value
