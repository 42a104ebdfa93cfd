"""Python layer objects over the C ABI (thin ctypes veneer, no computation here).

Buffers may be torch tensors (any device), numpy arrays or raw integer addresses; the library
itself decides per pointer whether staging is needed.  ``stream`` arguments are raw
``cudaStream_t`` values (e.g. ``torch.cuda.current_stream().cuda_stream``).
"""
from __future__ import annotations

import ctypes as C

from . import capi

DTYPES = {"float32": capi.DTYPE_FLOAT32, "float16": capi.DTYPE_FLOAT16,
          "qint8_rowwise_f32": capi.DTYPE_QINT8_F32, "qint8_rowwise_f16": capi.DTYPE_QINT8_F16,
          "quint8_rowwise_f32": capi.DTYPE_QUINT8_F32, "quint8_rowwise_f16": capi.DTYPE_QUINT8_F16}
POOLING = {"concatenate": capi.POOL_CONCATENATE, "sum": capi.POOL_SUM, "mean": capi.POOL_MEAN,
           "weighted_sum": capi.POOL_WEIGHTED_SUM, "weighted_mean": capi.POOL_WEIGHTED_MEAN}


def address(buf) -> int | None:
    if buf is None:
        return None
    if isinstance(buf, int):
        return buf
    if hasattr(buf, "data_ptr"):
        return buf.data_ptr()
    return buf.ctypes.data


def _dtype(x) -> int:
    return DTYPES[x] if isinstance(x, str) else int(x)


class ExecutionContext:
    """nve_context_t bound to a layer or table."""

    def __init__(self, handle: C.c_void_p):
        self.handle = handle

    def wait(self) -> None:
        capi.check(capi.lib.nve_context_wait(self.handle))

    def destroy(self) -> None:
        if self.handle:
            capi.check(capi.lib.nve_context_destroy(self.handle))
            self.handle = None


class _Layer:
    handle: C.c_void_p

    def create_execution_context(self, lookup_stream: int | None = None,
                                 modify_stream: int | None = None) -> ExecutionContext:
        h = C.c_void_p()
        capi.check(capi.lib.nve_layer_create_execution_context(
            self.handle, C.byref(h), lookup_stream, modify_stream, None, None))
        return ExecutionContext(h)

    def lookup(self, ctx: ExecutionContext, num_keys: int, keys, output, output_stride: int,
               hitmask=None, want_hitrate: bool = False):
        hr = (C.c_float * 4)()
        capi.check(capi.lib.nve_layer_lookup(self.handle, ctx.handle, num_keys, address(keys),
                                             address(output), output_stride, address(hitmask),
                                             hr if want_hitrate else None))
        return hr[0] if want_hitrate else None

    def lookup_pooled(self, ctx: ExecutionContext, num_keys: int, keys, output, output_stride: int,
                      pooling: str, output_type, *, csr_offsets=None, num_csr_offsets: int = 0,
                      fixed_hotness: int = 0, weights=None, weight_type=capi.DTYPE_UNKNOWN,
                      hitmask=None, want_hitrate: bool = False):
        hr = (C.c_float * 4)()
        capi.check(capi.lib.nve_layer_lookup_pooled(
            self.handle, ctx.handle, num_keys, address(keys), address(output), output_stride,
            address(hitmask), POOLING[pooling],
            capi.SPARSE_CSR if csr_offsets is not None else capi.SPARSE_FIXED,
            address(csr_offsets), num_csr_offsets, fixed_hotness, address(weights),
            _dtype(weight_type), _dtype(output_type), hr if want_hitrate else None))
        return hr[0] if want_hitrate else None

    def insert(self, ctx, num_keys, keys, value_stride, value_size, values, table_id=0):
        capi.check(capi.lib.nve_layer_insert(self.handle, ctx.handle, num_keys, address(keys),
                                             value_stride, value_size, address(values), table_id))

    def update(self, ctx, num_keys, keys, value_stride, value_size, values, table_id=0):
        capi.check(capi.lib.nve_layer_update(self.handle, ctx.handle, num_keys, address(keys),
                                             value_stride, value_size, address(values), table_id))

    def accumulate(self, ctx, num_keys, keys, value_stride, value_size, values, value_type,
                   table_id=0):
        capi.check(capi.lib.nve_layer_accumulate(self.handle, ctx.handle, num_keys, address(keys),
                                                 value_stride, value_size, address(values),
                                                 _dtype(value_type), table_id))

    def clear(self, ctx):
        capi.check(capi.lib.nve_layer_clear(self.handle, ctx.handle))

    def erase(self, ctx, num_keys, keys, table_id=0):
        capi.check(capi.lib.nve_layer_erase(self.handle, ctx.handle, num_keys, address(keys), table_id))

    def destroy(self):
        if self.handle:
            capi.check(capi.lib.nve_layer_destroy(self.handle))
            self.handle = None


class GPUEmbeddingLayer(_Layer):
    """Dense table resident in HBM (nve_gpu_embedding_layer_create)."""

    def __init__(self, embedding_table, num_embeddings: int, embedding_width_in_bytes: int,
                 value_dtype, *, key_type: int = capi.KEY_INT64, device_id: int = 0,
                 default_row_index: int = -1, layer_name: str = "gpu_layer"):
        cfg = capi.lib.nve_gpu_embedding_layer_config_default()
        self._name = layer_name.encode()
        cfg.layer_name = self._name
        cfg.device_id = device_id
        cfg.embedding_table = address(embedding_table)
        cfg.num_embeddings = num_embeddings
        cfg.embedding_width_in_bytes = embedding_width_in_bytes
        cfg.value_dtype = _dtype(value_dtype)
        cfg.default_row_index = default_row_index
        self._keepalive = embedding_table
        h = C.c_void_p()
        capi.check(capi.lib.nve_gpu_embedding_layer_create(C.byref(h), key_type, C.byref(cfg), None))
        self.handle = h


class GpuTable:
    """Set-associative GPU cache table (nve_gpu_table_create)."""

    def __init__(self, cache_size: int, row_size_in_bytes: int, value_dtype, *,
                 key_type: int = capi.KEY_INT64, device_id: int = 0, uvm_table=None,
                 uvm_num_rows: int = 0, count_misses: bool = True,
                 max_modify_size: int = 1 << 20, invalid_key: int = -1,
                 kernel_mode_type: int = 0, kernel_mode_value: int = 0,
                 modify_on_gpu: bool = True, data_storage_on_host: bool = False):
        cfg = capi.lib.nve_gpu_table_config_default()
        cfg.modify_on_gpu = int(modify_on_gpu)            # False: replacement decided on the host
        cfg.data_storage_on_host = int(data_storage_on_host)   # True: cached rows in pinned host memory
        cfg.kernel_mode_type = kernel_mode_type     # 0 dynamic, 1 fused lookup, 2 sort-gather, 3 pipeline
        cfg.kernel_mode_value = kernel_mode_value
        cfg.device_id = device_id
        cfg.cache_size = cache_size
        cfg.row_size_in_bytes = row_size_in_bytes
        cfg.uvm_table = address(uvm_table)
        cfg.uvm_num_rows = uvm_num_rows
        cfg.count_misses = int(count_misses)
        cfg.max_modify_size = max_modify_size
        cfg.value_dtype = _dtype(value_dtype)
        cfg.invalid_key = invalid_key
        self._keepalive = uvm_table
        self.key_type = key_type
        h = C.c_void_p()
        capi.check(capi.lib.nve_gpu_table_create(C.byref(h), key_type, C.byref(cfg), None))
        self.handle = h

    def create_execution_context(self, lookup_stream=None, modify_stream=None) -> ExecutionContext:
        h = C.c_void_p()
        capi.check(capi.lib.nve_table_create_execution_context(
            self.handle, C.byref(h), lookup_stream, modify_stream, None, None))
        return ExecutionContext(h)

    def find(self, ctx, n, keys, hit_mask, value_stride, values):
        capi.check(capi.lib.nve_table_find(self.handle, ctx.handle, n, address(keys),
                                           address(hit_mask), value_stride, address(values), None))

    def insert(self, ctx, n, keys, value_stride, value_size, values):
        capi.check(capi.lib.nve_table_insert(self.handle, ctx.handle, n, address(keys),
                                             value_stride, value_size, address(values)))

    def update(self, ctx, n, keys, value_stride, value_size, values):
        capi.check(capi.lib.nve_table_update(self.handle, ctx.handle, n, address(keys),
                                             value_stride, value_size, address(values)))

    def update_accumulate(self, ctx, n, keys, update_stride, update_size, updates, update_dtype):
        capi.check(capi.lib.nve_table_update_accumulate(
            self.handle, ctx.handle, n, address(keys), update_stride, update_size,
            address(updates), _dtype(update_dtype)))

    def clear(self, ctx):
        capi.check(capi.lib.nve_table_clear(self.handle, ctx.handle))

    def erase(self, ctx, n, keys):
        capi.check(capi.lib.nve_table_erase(self.handle, ctx.handle, n, address(keys)))

    def reset_lookup_counter(self, ctx):
        capi.check(capi.lib.nve_table_reset_lookup_counter(self.handle, ctx.handle))

    def get_lookup_counter(self, ctx) -> int:
        v = C.c_int64()
        capi.check(capi.lib.nve_table_get_lookup_counter(self.handle, ctx.handle, C.byref(v)))
        return v.value

    def destroy(self):
        if self.handle:
            capi.check(capi.lib.nve_table_destroy(self.handle))
            self.handle = None


class LinearUVMEmbeddingLayer(_Layer):
    """GPU cache in front of a linear table in host / managed / device memory
    (nve_linear_uvm_layer_create).  The layer keeps its GpuTable alive."""

    def __init__(self, gpu_table: GpuTable, *, default_row_index: int = -1,
                 layer_name: str = "linear_uvm_layer", insert_heuristic="never",
                 min_insert_freq_gpu: int | None = None, min_insert_size_gpu: int | None = None):
        """insert_heuristic: "never" (this wrapper's default: the cache holds what the caller
        inserts), "default" (the C ABI's default: NULL handle, threshold 0.75) or a float threshold
        for the default heuristic.  Automatic inserts need a table created with count_misses."""
        cfg = capi.lib.nve_linear_uvm_layer_config_default()
        self._name = layer_name.encode()
        cfg.layer_name = self._name
        cfg.default_row_index = default_row_index
        if min_insert_freq_gpu is not None:
            cfg.min_insert_freq_gpu = min_insert_freq_gpu
        if min_insert_size_gpu is not None:
            cfg.min_insert_size_gpu = min_insert_size_gpu
        heuristic = C.c_void_p()
        if insert_heuristic == "never":
            capi.check(capi.lib.nve_heuristic_create_never(C.byref(heuristic)))
        elif insert_heuristic != "default":
            thr = (C.c_float * 1)(float(insert_heuristic))
            capi.check(capi.lib.nve_heuristic_create_default(C.byref(heuristic), thr, 1))
        cfg.insert_heuristic = heuristic
        self.gpu_table = gpu_table
        h = C.c_void_p()
        try:
            capi.check(capi.lib.nve_linear_uvm_layer_create(C.byref(h), gpu_table.key_type,
                                                            C.byref(cfg), gpu_table.handle, None))
        finally:
            if heuristic:                       # the layer copied it
                capi.check(capi.lib.nve_heuristic_destroy(heuristic))
        self.handle = h
