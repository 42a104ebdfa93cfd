"""Small helpers for driving libnve_b200 through its C ABI from tests (torch supplies device memory)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from nv_embedding_cache_b200 import capi

DT = {"f32": capi.DTYPE_FLOAT32, "f16": capi.DTYPE_FLOAT16, "qint8_f32": capi.DTYPE_QINT8_F32,
      "qint8_f16": capi.DTYPE_QINT8_F16, "quint8_f32": capi.DTYPE_QUINT8_F32,
      "quint8_f16": capi.DTYPE_QUINT8_F16}
POOL = {"concat": capi.POOL_CONCATENATE, "sum": capi.POOL_SUM, "mean": capi.POOL_MEAN,
        "wsum": capi.POOL_WEIGHTED_SUM, "wmean": capi.POOL_WEIGHTED_MEAN}
NP_OUT = {"f32": np.float32, "f16": np.float16}


def ptr(x):
    """Address of a numpy array, torch tensor, or None."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    return x.data_ptr()


class Context:
    def __init__(self, handle):
        self.h = handle

    def wait(self):
        capi.check(capi.lib.nve_context_wait(self.h))

    def destroy(self):
        if self.h:
            capi.check(capi.lib.nve_context_destroy(self.h))
            self.h = None


class GpuLayer:
    """nve_gpu_embedding_layer_create + one execution context on the default stream."""

    def __init__(self, table_dev, num_rows, row_bytes, value_dtype, key_type=capi.KEY_INT64,
                 default_row=-1, device=0):
        cfg = capi.lib.nve_gpu_embedding_layer_config_default()
        cfg.layer_name = b"test"
        cfg.device_id = device
        cfg.embedding_table = ptr(table_dev)
        cfg.num_embeddings = num_rows
        cfg.embedding_width_in_bytes = row_bytes
        cfg.value_dtype = DT[value_dtype]
        cfg.default_row_index = default_row
        self._table = table_dev
        h = C.c_void_p()
        capi.check(capi.lib.nve_gpu_embedding_layer_create(C.byref(h), key_type, C.byref(cfg), None))
        self.h = h
        c = C.c_void_p()
        capi.check(capi.lib.nve_layer_create_execution_context(self.h, C.byref(c), None, None, None, None))
        self.ctx = Context(c)

    def lookup(self, keys, out, stride):
        hr = C.c_float(-1)
        st = capi.lib.nve_layer_lookup(self.h, self.ctx.h, _n(keys), ptr(keys), ptr(out), stride, None,
                                       C.byref(hr))
        capi.check(st)
        return hr.value

    def lookup_pooled(self, keys, out, stride, pooling, *, offsets=None, hotness=0, weights=None,
                      weight_dtype="f32", out_dtype="f32", num_keys=None):
        hr = C.c_float(-1)
        st = capi.lib.nve_layer_lookup_pooled(
            self.h, self.ctx.h, _n(keys) if num_keys is None else num_keys, ptr(keys), ptr(out),
            stride, None, POOL[pooling], capi.SPARSE_CSR if offsets is not None else capi.SPARSE_FIXED,
            ptr(offsets), _n(offsets) if offsets is not None else 0, hotness, ptr(weights),
            DT[weight_dtype], DT[out_dtype], C.byref(hr))
        capi.check(st)
        return hr.value

    def update(self, keys, values, stride, size):
        capi.check(capi.lib.nve_layer_update(self.h, self.ctx.h, _n(keys), ptr(keys), stride, size,
                                             ptr(values), 0))

    def accumulate(self, keys, values, stride, size, value_dtype):
        capi.check(capi.lib.nve_layer_accumulate(self.h, self.ctx.h, _n(keys), ptr(keys), stride,
                                                 size, ptr(values), DT[value_dtype], 0))

    def close(self):
        self.ctx.wait()
        self.ctx.destroy()
        if self.h:
            capi.check(capi.lib.nve_layer_destroy(self.h))
            self.h = None


def _n(x):
    if x is None:
        return 0
    if isinstance(x, np.ndarray):
        return x.size
    return x.numel()


def to_dev(torch, a: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-30))) if a.size else 0.0


# ---- GPU cache table helpers --------------------------------------------------------------------
def device_read(ptr_value: int, nbytes: int) -> np.ndarray:
    """Copy nbytes from a raw device address to a numpy buffer (UVA memcpy through cuda-python)."""
    from cuda import cudart
    out = np.empty(nbytes, dtype=np.uint8)
    (err,) = cudart.cudaDeviceSynchronize()
    assert int(err) == 0, err
    (err,) = cudart.cudaMemcpy(out.ctypes.data, ptr_value, nbytes, cudart.cudaMemcpyKind.cudaMemcpyDefault)
    assert int(err) == 0, err
    return out


class CacheTable:
    """nve_gpu_table_create + one execution context; state readers for parity checks."""

    def __init__(self, cache_bytes, row_bytes, value_dtype="f16", key_dtype=np.int64, backing=None,
                 backing_rows=0, max_modify=1 << 20, sentinel=-1, modify_on_gpu=True,
                 data_storage_on_host=False):
        from nv_embedding_cache_b200.layers import GpuTable
        self.key_dtype = np.dtype(key_dtype)
        self.row_bytes = row_bytes
        kt = capi.KEY_INT64 if self.key_dtype.itemsize == 8 else capi.KEY_INT32
        self.table = GpuTable(cache_bytes, row_bytes, DT[value_dtype], key_type=kt, uvm_table=backing,
                              uvm_num_rows=backing_rows, max_modify_size=max_modify,
                              invalid_key=sentinel, modify_on_gpu=modify_on_gpu,
                              data_storage_on_host=data_storage_on_host)
        self.ctx = self.table.create_execution_context()
        view = capi.CacheData()
        capi.check(capi.lib.nve_b200_gpu_table_get_cache_data(self.table.handle, self.ctx.handle,
                                                              C.byref(view)))
        self.view = view
        self.num_sets = view.num_sets
        self.sentinel = sentinel

    def tags(self) -> np.ndarray:
        raw = device_read(self.view.tags_ptr, self.num_sets * 8 * self.key_dtype.itemsize)
        return raw.view(self.key_dtype).astype(np.int64).reshape(self.num_sets, 8)

    def data(self) -> np.ndarray:
        raw = device_read(self.view.cache_ptr, self.num_sets * 8 * self.row_bytes)
        return raw.reshape(self.num_sets, 8, self.row_bytes)

    def counters(self) -> np.ndarray:
        p, q = C.c_void_p(), C.c_void_p()
        capi.check(capi.lib.nve_b200_gpu_table_get_policy_state(self.table.handle, C.byref(p), C.byref(q)))
        return device_read(p.value, self.num_sets * 8 * 4).view(np.float32).reshape(self.num_sets, 8)

    def keys_of(self, a):
        return np.ascontiguousarray(a, dtype=self.key_dtype)

    def insert(self, keys, values):
        keys = self.keys_of(keys)
        self.table.insert(self.ctx, keys.size, keys, values.strides[0], self.row_bytes, values)
        self.ctx.wait()

    def insert_from_backing(self, keys):
        keys = self.keys_of(keys)
        capi.check(capi.lib.nve_b200_gpu_table_insert_from_backing(self.table.handle, self.ctx.handle,
                                                                   keys.size, keys.ctypes.data))
        self.ctx.wait()

    def find(self, keys, out, hit_mask=None):
        keys = self.keys_of(keys)
        self.table.reset_lookup_counter(self.ctx)
        self.table.find(self.ctx, keys.size, keys, hit_mask, out.strides[0] if out is not None else 0, out)
        self.ctx.wait()
        v = self.table.get_lookup_counter(self.ctx)
        self.ctx.wait()
        return self.table_counter()

    def table_counter(self) -> int:
        v = C.c_int64(-1)
        capi.check(capi.lib.nve_table_get_lookup_counter(self.table.handle, self.ctx.handle, C.byref(v)))
        self.ctx.wait()
        return v.value

    def update(self, keys, values):
        keys = self.keys_of(keys)
        self.table.update(self.ctx, keys.size, keys, values.strides[0], self.row_bytes, values)
        self.ctx.wait()

    def update_accumulate(self, keys, updates, dtype):
        keys = self.keys_of(keys)
        self.table.update_accumulate(self.ctx, keys.size, keys, updates.strides[0], self.row_bytes,
                                     updates, DT[dtype])
        self.ctx.wait()

    def erase(self, keys):
        keys = self.keys_of(keys)
        self.table.erase(self.ctx, keys.size, keys)
        self.ctx.wait()

    def clear(self):
        self.table.clear(self.ctx)
        self.ctx.wait()

    def close(self):
        self.ctx.wait()
        self.ctx.destroy()
        self.table.destroy()
