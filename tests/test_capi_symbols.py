"""CPU checks of the C-ABI library: it loads, and it exports every symbol include/*.h declares."""
import ctypes as C
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    names = set()
    for hdr in sorted((ROOT / "include").glob("*.h")):
        text = hdr.read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"NVE_C_API\s+[\w\s\*]+?\b(nve_\w+)\s*\(", text):
            names.add(m.group(1))
    return names


def test_every_declared_symbol_is_exported(capi):
    declared = _declared_symbols()
    assert len(declared) >= 50
    missing = [n for n in sorted(declared) if not hasattr(capi.lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"
    unbound = sorted(declared - set(capi.PROTOTYPES))
    assert not unbound, f"no ctypes prototype for: {unbound}"


def test_versions_and_defaults(capi):
    a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
    assert capi.lib.nve_version(C.byref(a), C.byref(b), C.byref(c)) == 0
    assert (a.value, b.value) == (26, 9)
    assert capi.lib.nve_abi_version(C.byref(a), C.byref(b)) == 0
    assert (a.value, b.value) == (1, 0)
    t = capi.lib.nve_gpu_table_config_default()
    assert (t.count_misses, t.max_modify_size, t.uvm_cpu_accumulate, t.modify_on_gpu, t.invalid_key) == \
        (1, 1 << 20, 1, 1, -1)
    g = capi.lib.nve_gpu_embedding_layer_config_default()
    assert g.default_row_index == -1 and g.value_dtype == 0
    u = capi.lib.nve_linear_uvm_layer_config_default()
    assert u.min_insert_size_gpu == 1 << 16 and u.default_row_index == -1


def test_null_handles_are_invalid_argument(capi):
    st = capi.lib.nve_layer_lookup(None, None, 0, None, None, 0, None, None)
    assert st == capi.NVE_ERROR_INVALID_ARGUMENT
    assert "must not be NULL" in capi.last_error()
    assert capi.lib.nve_context_wait(None) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert capi.lib.nve_table_find(None, None, 0, None, None, 0, None, None) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert capi.lib.nve_version(None, None, None) == capi.NVE_ERROR_INVALID_ARGUMENT
    out = C.c_void_p()
    assert capi.lib.nve_create_table_factory(C.byref(out), b"plugin.so", b"{}") == capi.NVE_ERROR_NOT_IMPLEMENTED
    assert capi.lib.nve_gpu_embedding_layer_create(None, 1, None, None) == capi.NVE_ERROR_INVALID_ARGUMENT


def test_heuristic_handles(capi):
    h = C.c_void_p()
    assert capi.lib.nve_heuristic_create_never(C.byref(h)) == 0 and h.value
    assert capi.lib.nve_heuristic_destroy(h) == 0
    assert capi.lib.nve_heuristic_create_default(C.byref(h), None, 0) == 0
    assert capi.lib.nve_heuristic_destroy(h) == 0
    assert capi.lib.nve_heuristic_destroy(None) == capi.NVE_ERROR_INVALID_ARGUMENT


def test_kernel_level_entry_points_check_arguments_before_any_gpu_work(capi):
    """No GPU here: these calls must be answered from the argument checks alone."""
    inv = capi.NVE_ERROR_INVALID_ARGUMENT
    n = C.c_int64(0)
    assert capi.lib.nve_b200_pooling_backprop(None, 8, None, None, 64, 64, capi.POOL_SUM, capi.SPARSE_CSR,
                                              None, 1, 0, None, None, None, 64, C.byref(n), None) == inv
    assert capi.lib.nve_b200_dedup_grads_f16(None, None, 64, 64, 8, None, None, None, None, 64, None) == inv
    assert capi.lib.nve_b200_dedup_grads(None, None, 64, 64, 8, None, None, None, None, None, 64, 0, 0, 1.0,
                                         None) == inv
    assert capi.lib.nve_b200_deduper_dedup(None, None, 0, None, None, None, None, None, None, None, 0) == inv
    assert capi.lib.nve_b200_managed_block_create(None, 1 << 20, None, 0) == inv
    assert capi.lib.nve_b200_managed_block_destroy(None) == 0            # destroying nothing is fine
    assert capi.lib.nve_b200_scatter_rows(None, 64, None, 64, 64, None, 0, None) == 0   # zero rows: nothing to do
    assert capi.lib.nve_b200_scatter_rows(None, 64, None, 64, 64, None, 4, None) == inv
    assert "NULL" in capi.last_error()


def test_failed_creators_leave_null_and_bad_key_types_are_rejected(capi):
    """What the reference's tests/c_api/c_api_malformed_input_test.cpp:97-110 and
    c_api_handle_lifecycle_test.cpp:150-173 ask of creators: an unsupported key type is an invalid
    argument, and a creator that fails never leaves a stale handle behind."""
    lib = capi.lib
    cfg = lib.nve_gpu_table_config_default()
    cfg.cache_size, cfg.row_size_in_bytes = 1 << 20, 128
    table = C.c_void_p()
    assert lib.nve_gpu_table_create(C.byref(table), 99, C.byref(cfg), None) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert table.value is None and "Unsupported key type" in capi.last_error()
    assert lib.nve_gpu_table_create(None, capi.KEY_INT64, C.byref(cfg), None) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert lib.nve_gpu_table_create(C.byref(table), capi.KEY_INT64, None, None) == capi.NVE_ERROR_INVALID_ARGUMENT
    for call in (lambda h: lib.nve_create_table_factory(C.byref(h), b"nonexistent_plugin_xyz.so", b"{}"),
                 lambda h: lib.nve_table_factory_produce(None, 0, b"not valid json", C.byref(h)),
                 lambda h: lib.nve_hierarchical_layer_create(C.byref(h), capi.KEY_INT64, None, None, 0, None),
                 lambda h: lib.nve_host_embedding_layer_create(C.byref(h), capi.KEY_INT64, None, None, None)):
        sentinel = C.c_void_p(1)
        assert call(sentinel) == capi.NVE_ERROR_NOT_IMPLEMENTED
        assert sentinel.value is None
    # getters answer NULL handles and NULL outputs with a status, never a crash
    for name in ("nve_table_get_device_id", "nve_table_get_max_row_size", "nve_table_get_key_size"):
        assert getattr(lib, name)(None, None) == capi.NVE_ERROR_INVALID_ARGUMENT


def test_thread_pool_lifecycle_and_malformed_configurations(capi):
    """After the reference's tests/c_api/c_api_threadpool_test.cpp: create with a valid configuration,
    num_workers reports it, destroy succeeds; malformed JSON and non-object JSON are statuses, not
    exceptions; NULL arguments are invalid."""
    lib, inv = capi.lib, capi.NVE_ERROR_INVALID_ARGUMENT
    pool = C.c_void_p()
    assert lib.nve_thread_pool_create(C.byref(pool), b'{"name": "simple", "num_workers": 3}') == 0
    assert pool.value
    n = C.c_int64(-1)
    assert lib.nve_thread_pool_num_workers(pool, C.byref(n)) == 0 and n.value == 3
    assert lib.nve_thread_pool_num_workers(None, C.byref(n)) == inv
    assert lib.nve_thread_pool_num_workers(pool, None) == inv
    assert lib.nve_thread_pool_destroy(pool) == 0
    assert lib.nve_thread_pool_destroy(None) == inv
    for bad in (b"{not valid json", b"[1, 2, 3]", b"42", b'{"num_workers": "three"}', b'{"num_workers": -1}',
                b'{"num_workers": 2.5}', b'{"num_workers": 3} trailing', b'{"a": [1, 2,}'):
        h = C.c_void_p(1)
        assert lib.nve_thread_pool_create(C.byref(h), bad) == inv, bad
        assert h.value is None
    assert lib.nve_thread_pool_create(None, b"{}") == inv
    assert lib.nve_thread_pool_create(C.byref(pool), None) == inv
    # nested values and escapes are read past; without num_workers the pool takes the default size
    ok = b'{"name": "simple \\"quoted\\"", "extra": {"list": [1, 2.5e3, true, null, {"x": []}]}}'
    assert lib.nve_thread_pool_create(C.byref(pool), ok) == 0
    assert lib.nve_thread_pool_num_workers(pool, C.byref(n)) == 0 and n.value >= 1
    assert lib.nve_thread_pool_destroy(pool) == 0
    assert lib.nve_configure_default_thread_pool(b"{oops") == inv
    assert lib.nve_configure_default_thread_pool(None) == inv
