"""ctypes binding of libnve_b200.so — the same calls a C program makes through nve_c_api.h.

Loading fails loudly when the library has not been built (``python -m nv_embedding_cache_b200.build``);
there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# NVE_B200_LIBRARY: another build of the library to load, e.g. the checked one
# (libnve_b200_checked.so, `python -m nv_embedding_cache_b200.build --bounds-check`)
PACKAGE_DIR = Path(__file__).resolve().parent
_LIB_PATH = Path(os.environ.get("NVE_B200_LIBRARY") or Path(__file__).resolve().parent / "libnve_b200.so")

# ---- enums (include/nve_c_api.h) -------------------------------------------------------------
NVE_SUCCESS, NVE_ERROR_INVALID_ARGUMENT, NVE_ERROR_CUDA, NVE_ERROR_RUNTIME = 0, 1, 2, 3
NVE_ERROR_NOT_IMPLEMENTED, NVE_ERROR_OUT_OF_MEMORY = 4, 5
DTYPE_UNKNOWN, DTYPE_FLOAT32, DTYPE_BFLOAT16, DTYPE_FLOAT16 = 0, 1, 2, 3
DTYPE_QINT8_F32, DTYPE_QINT8_F16, DTYPE_QUINT8_F32, DTYPE_QUINT8_F16 = 7, 8, 9, 10
SPARSE_FIXED, SPARSE_CSR = 0, 1
POOL_CONCATENATE, POOL_SUM, POOL_MEAN, POOL_WEIGHTED_SUM, POOL_WEIGHTED_MEAN = 0, 1, 2, 3, 4
KEY_INT32, KEY_INT64 = 0, 1

_vp, _i64, _i32, _u64 = C.c_void_p, C.c_int64, C.c_int32, C.c_uint64


class GpuTableConfig(C.Structure):
    _fields_ = [("device_id", _i32), ("cache_size", _u64), ("row_size_in_bytes", _i64),
                ("uvm_table", _vp), ("count_misses", C.c_int), ("max_modify_size", _i64),
                ("value_dtype", _i32), ("private_stream", _vp), ("disable_uvm_update", C.c_int),
                ("uvm_cpu_accumulate", C.c_int), ("data_storage_on_host", C.c_int),
                ("modify_on_gpu", C.c_int), ("kernel_mode_type", _u64),
                ("kernel_mode_value", _u64), ("invalid_key", _i64), ("uvm_num_rows", _i64)]


class GpuEmbeddingLayerConfig(C.Structure):
    _fields_ = [("layer_name", C.c_char_p), ("device_id", _i32), ("embedding_table", _vp),
                ("num_embeddings", _i64), ("embedding_width_in_bytes", _i64),
                ("value_dtype", _i32), ("default_row_index", _i64)]


class LinearUvmLayerConfig(C.Structure):
    _fields_ = [("layer_name", C.c_char_p), ("insert_heuristic", _vp),
                ("min_insert_freq_gpu", _i64), ("min_insert_size_gpu", _i64),
                ("default_row_index", _i64)]


class CacheData(C.Structure):
    _fields_ = [("cache_ptr", _vp), ("tags_ptr", _vp), ("num_sets", C.c_uint32),
                ("row_size_in_bytes", _u64), ("count_misses", C.c_bool), ("misses", _vp)]


class PoolArgs(C.Structure):
    _fields_ = [("table", _vp), ("num_rows", _i64), ("row_stride", _i64), ("value_dtype", _i32),
                ("row_width", _i64), ("default_row_index", _i64), ("cache", C.POINTER(CacheData)),
                ("key_type", C.c_int), ("keys", _vp), ("num_keys", _i64),
                ("pooling_type", C.c_int), ("sparse_type", C.c_int), ("csr_offsets", _vp),
                ("offset_bytes", _i32), ("num_bags", _i64), ("fixed_hotness", _i64),
                ("weights", _vp), ("weight_dtype", _i32), ("output", _vp),
                ("output_stride", _i64), ("output_dtype", _i32),
                ("shard_tables", C.POINTER(_vp)), ("num_shards", _i32)]


class GatherArgs(C.Structure):
    _fields_ = [("table", _vp), ("num_rows", _i64), ("row_stride", _i64), ("value_dtype", _i32),
                ("row_width", _i64), ("default_row_index", _i64), ("cache", C.POINTER(CacheData)),
                ("key_type", C.c_int), ("keys", _vp), ("num_keys", _i64), ("output", _vp),
                ("output_stride", _i64), ("output_dtype", _i32), ("row_copy_bytes", _i64),
                ("hit_mask", _vp), ("miss_count", _vp), ("miss_positions", _vp),
                ("miss_keys", _vp), ("miss_list_len", _vp)]


SHARD_PEER, SHARD_EXCHANGE = 0, 1

# transport callbacks of the exchange form (nve_b200_exchange_ops_t)
ALL_GATHER_U32_FN = C.CFUNCTYPE(C.c_int, _vp, _vp, _vp, _i64, _vp)
ALL_TO_ALL_V_FN = C.CFUNCTYPE(C.c_int, _vp, _vp, C.POINTER(_i64), _vp, C.POINTER(_i64), _i64, _vp)


class ExchangeOps(C.Structure):
    _fields_ = [("user", _vp), ("all_gather_u32", ALL_GATHER_U32_FN), ("all_to_all_v", ALL_TO_ALL_V_FN)]


class ShardedTableConfig(C.Structure):
    _fields_ = [("world", _i32), ("rank", _i32), ("device_id", _i32), ("mode", C.c_int),
                ("local_shard", _vp), ("local_rows", _i64), ("row_stride", _i64), ("value_dtype", _i32),
                ("row_width", _i64), ("key_type", C.c_int), ("default_row_index", _i64),
                ("max_keys", _i64), ("peer_shards", C.POINTER(_vp)), ("nccl_unique_id", _vp),
                ("exchange_ops", C.POINTER(ExchangeOps)), ("hot_capacity", _i64),
                ("exchange_timeout_ms", _i64)]


class ShardedLookup(C.Structure):
    _fields_ = [("keys", _vp), ("num_keys", _i64), ("pooling_type", C.c_int), ("sparse_type", C.c_int),
                ("csr_offsets", _vp), ("offset_bytes", _i32), ("num_bags", _i64), ("fixed_hotness", _i64),
                ("weights", _vp), ("weight_dtype", _i32), ("output", _vp), ("output_stride", _i64),
                ("output_dtype", _i32)]


class NveError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"nve status {status}: {message}")
        self.status = status
        self.message = message


def _load() -> C.CDLL:
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m nv_embedding_cache_b200.build` "
            "(there is no CPU fallback)")
    return C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)


lib = _load()

# name -> (restype, argtypes); every symbol include/*.h declares.
PROTOTYPES = {
    "nve_get_last_error": (_i32, [C.POINTER(C.c_char_p)]),
    "nve_gpu_table_config_default": (GpuTableConfig, []),
    "nve_gpu_embedding_layer_config_default": (GpuEmbeddingLayerConfig, []),
    "nve_linear_uvm_layer_config_default": (LinearUvmLayerConfig, []),
    "nve_hierarchical_layer_config_default": (None, None),
    "nve_host_embedding_layer_config_default": (None, None),
    "nve_overflow_policy_config_default": (None, None),
    "nve_host_table_config_default": (None, None),
    "nve_version": (_i32, [C.POINTER(_i32)] * 3),
    "nve_abi_version": (_i32, [C.POINTER(_i32)] * 2),
    "nve_thread_pool_create": (_i32, [C.POINTER(_vp), C.c_char_p]),
    "nve_thread_pool_destroy": (_i32, [_vp]),
    "nve_thread_pool_num_workers": (_i32, [_vp, C.POINTER(_i64)]),
    "nve_configure_default_thread_pool": (_i32, [C.c_char_p]),
    "nve_heuristic_create_default": (_i32, [C.POINTER(_vp), _vp, _i64]),
    "nve_heuristic_create_never": (_i32, [C.POINTER(_vp)]),
    "nve_heuristic_destroy": (_i32, [_vp]),
    "nve_context_destroy": (_i32, [_vp]),
    "nve_context_wait": (_i32, [_vp]),
    "nve_context_get_lookup_stream": (_i32, [_vp, C.POINTER(_vp)]),
    "nve_context_get_modify_stream": (_i32, [_vp, C.POINTER(_vp)]),
    "nve_gpu_table_create": (_i32, [C.POINTER(_vp), C.c_int, C.POINTER(GpuTableConfig), _vp]),
    "nve_table_destroy": (_i32, [_vp]),
    "nve_table_find": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _vp]),
    "nve_table_insert": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _vp]),
    "nve_table_update": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _vp]),
    "nve_table_update_accumulate": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _vp, _i32]),
    "nve_table_clear": (_i32, [_vp, _vp]),
    "nve_table_erase": (_i32, [_vp, _vp, _i64, _vp]),
    "nve_table_create_execution_context": (_i32, [_vp, C.POINTER(_vp), _vp, _vp, _vp, _vp]),
    "nve_table_get_device_id": (_i32, [_vp, C.POINTER(_i32)]),
    "nve_table_get_max_row_size": (_i32, [_vp, C.POINTER(_i64)]),
    "nve_table_get_key_size": (_i32, [_vp, C.POINTER(_i64)]),
    "nve_table_reset_lookup_counter": (_i32, [_vp, _vp]),
    "nve_table_get_lookup_counter": (_i32, [_vp, _vp, C.POINTER(_i64)]),
    "nve_create_table_factory": (_i32, [C.POINTER(_vp), C.c_char_p, C.c_char_p]),
    "nve_table_factory_destroy": (_i32, [_vp]),
    "nve_table_factory_produce": (_i32, [_vp, _i64, C.c_char_p, C.POINTER(_vp)]),
    "nve_gpu_embedding_layer_create": (_i32, [C.POINTER(_vp), C.c_int,
                                               C.POINTER(GpuEmbeddingLayerConfig), _vp]),
    "nve_linear_uvm_layer_create": (_i32, [C.POINTER(_vp), C.c_int,
                                            C.POINTER(LinearUvmLayerConfig), _vp, _vp]),
    "nve_hierarchical_layer_create": (_i32, [C.POINTER(_vp), C.c_int, _vp, _vp, _i64, _vp]),
    "nve_host_embedding_layer_create": (_i32, [C.POINTER(_vp), C.c_int, _vp, _vp, _vp]),
    "nve_layer_destroy": (_i32, [_vp]),
    "nve_layer_lookup": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _vp]),
    "nve_layer_lookup_pooled": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, C.c_int, C.c_int,
                                        _vp, _i64, _i64, _vp, _i32, _i32, _vp]),
    "nve_layer_insert": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _vp, _i64]),
    "nve_layer_update": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _vp, _i64]),
    "nve_layer_accumulate": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _vp, _i32, _i64]),
    "nve_layer_clear": (_i32, [_vp, _vp]),
    "nve_layer_erase": (_i32, [_vp, _vp, _i64, _vp, _i64]),
    "nve_layer_create_execution_context": (_i32, [_vp, C.POINTER(_vp), _vp, _vp, _vp, _vp]),
    "nve_layer_get_num_tables": (_i32, [_vp, C.POINTER(_i64)]),
    # kernel-level ABI (include/nve_b200_ops.h)
    "nve_b200_lookup_pool": (_i32, [C.POINTER(PoolArgs), _vp]),
    "nve_b200_gather_rows": (_i32, [C.POINTER(GatherArgs), _vp]),
    "nve_b200_gather_rows_sorted": (_i32, [C.POINTER(GatherArgs), _i64, _vp, C.POINTER(C.c_size_t), _vp]),
    "nve_b200_gpu_table_get_cache_data": (_i32, [_vp, _vp, C.POINTER(CacheData)]),
    "nve_b200_gpu_table_get_policy_state": (_i32, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "nve_b200_gpu_table_insert_from_backing": (_i32, [_vp, _vp, _i64, _vp]),
    "nve_b200_deduper_create": (_i32, [C.POINTER(_vp), C.c_int, _i64, _i64]),
    "nve_b200_deduper_destroy": (_i32, [_vp]),
    "nve_b200_deduper_dedup": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32]),
    "nve_b200_dedup_grads": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64,
                                     _i32, _i64, C.c_float, _vp]),
    "nve_b200_deduper_device_num_runs": (_i32, [_vp, C.POINTER(_vp)]),
    "nve_b200_shard_route_scratch_bytes": (_i32, [_i64, C.POINTER(_u64)]),
    "nve_b200_shard_route": (_i32, [C.c_int, _vp, _vp, _i64, _i32, _vp, _vp, _vp, _vp, _u64, _vp]),
    "nve_b200_shard_localise": (_i32, [C.c_int, _vp, _i64, _i32, _vp]),
    "nve_b200_shard_expand_slots": (_i32, [C.c_int, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "nve_b200_dedup_grads_static": (_i32, [C.c_int, _i64, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp,
                                            _vp, _vp, _i64, _i32, _i64, C.c_float, _vp]),
    "nve_b200_dedup_grads_status": (_i32, [C.POINTER(_i32)]),
    "nve_b200_registry_register": (_i32, [_vp, _vp, _i64, C.c_int, C.c_int]),
    "nve_b200_registry_unregister": (_i32, [_vp]),
    "nve_b200_registry_describe": (_i32, [_vp, C.POINTER(_i64), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "nve_b200_registry_size": (_i64, []),
    "nve_b200_registry_lookup": (_i32, [_vp, _i64, _vp, _vp, _vp]),
    "nve_b200_registry_lookup_pooled": (_i32, [_vp, _i64, _vp, _vp, C.c_int, _i64, _vp, C.c_int, _vp, _vp]),
    "nve_b200_nccl_unique_id": (_i32, [_vp]),
    "nve_b200_sharded_table_create": (_i32, [C.POINTER(_vp), C.POINTER(ShardedTableConfig)]),
    "nve_b200_sharded_table_destroy": (_i32, [_vp]),
    "nve_b200_sharded_table_lookup_pooled": (_i32, [_vp, C.POINTER(ShardedLookup), _vp]),
    "nve_b200_sharded_table_set_hot_keys": (_i32, [_vp, _vp, _i64, C.POINTER(_i64), _vp]),
    "nve_b200_sharded_table_stats": (_i32, [_vp, C.POINTER(_i64)]),
    "nve_b200_update_rows": (_i32, [_vp, _i64, _i64, _i32, _i64, C.c_int, _vp, _i64, _vp, _i64,
                                     C.c_int, C.c_int, _vp]),
    "nve_b200_dedup_grads_f16": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _vp]),
    "nve_b200_pooling_backprop": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, C.c_int, C.c_int, _vp, _i64, _i64,
                                          _vp, _vp, _vp, _i64, C.POINTER(_i64), _vp]),
    "nve_b200_scatter_rows": (_i32, [_vp, _i64, _vp, _i64, _i64, _vp, _i64, _vp]),
    "nve_b200_managed_block_create": (_i32, [C.POINTER(_vp), _u64, C.POINTER(_i32), _i32]),
    "nve_b200_managed_block_destroy": (_i32, [_vp]),
}

for _name, (_res, _args) in PROTOTYPES.items():
    _fn = getattr(lib, _name)  # AttributeError here means the library lacks a declared symbol
    if _args is not None:
        _fn.restype = _res
        _fn.argtypes = _args


def last_error() -> str:
    msg = C.c_char_p()
    lib.nve_get_last_error(C.byref(msg))
    return (msg.value or b"").decode(errors="replace")


def check(status: int) -> None:
    if status != NVE_SUCCESS:
        raise NveError(status, last_error())
