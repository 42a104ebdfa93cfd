"""Boundary behaviour of the table entry points of the C ABI on a GPU table, after the reference's
tests/c_api/c_api_boundary_test.cpp:139-256 (written there against a host table; the rules are those
of the shared entry points): zero keys are a no-op for every call, NULL keys with a positive count are
an invalid argument and change nothing, find works with any subset of its optional outputs, getters
refuse NULL outputs, and the lookup counter follows the misses after a reset."""
import ctypes as C

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi
from nve_helpers import CacheTable

pytestmark = pytest.mark.gpu

ROW = 64
INV = capi.NVE_ERROR_INVALID_ARGUMENT


@pytest.fixture()
def table(torch_cuda):
    t = CacheTable(64 * (64 + 8 * ROW + 32), ROW, key_dtype=np.int64)
    keys = np.arange(100, 140, dtype=np.int64)
    rows = np.random.default_rng(1).integers(0, 256, (keys.size, ROW), dtype=np.uint8)
    t.insert(keys, rows)
    yield t, keys, rows
    t.close()


def test_zero_keys_are_a_no_op(table):
    t, keys, rows = table
    lib, h, ctx = capi.lib, t.table.handle, t.ctx.handle
    before = t.tags().copy()
    assert lib.nve_table_find(h, ctx, 0, None, None, 0, None, None) == 0
    assert lib.nve_table_insert(h, ctx, 0, None, ROW, ROW, None) == 0
    assert lib.nve_table_update(h, ctx, 0, None, ROW, ROW, None) == 0
    assert lib.nve_table_update_accumulate(h, ctx, 0, None, ROW, ROW, None, capi.DTYPE_FLOAT32) == 0
    assert lib.nve_table_erase(h, ctx, 0, None) == 0
    t.ctx.wait()
    assert np.array_equal(t.tags(), before)


def test_null_keys_with_a_positive_count_are_rejected(table):
    t, keys, rows = table
    lib, h, ctx = capi.lib, t.table.handle, t.ctx.handle
    before = t.tags().copy()
    out = np.zeros((4, ROW), np.uint8)
    assert lib.nve_table_find(h, ctx, 4, None, None, ROW, out.ctypes.data, None) == INV
    assert "keys must not be null" in capi.last_error()
    assert lib.nve_table_insert(h, ctx, 4, None, ROW, ROW, out.ctypes.data) == INV
    assert lib.nve_table_update(h, ctx, 4, None, ROW, ROW, out.ctypes.data) == INV
    assert lib.nve_table_update_accumulate(h, ctx, 4, None, ROW, ROW, out.ctypes.data, capi.DTYPE_FLOAT32) == INV
    assert lib.nve_table_erase(h, ctx, 4, None) == INV
    t.ctx.wait()
    assert np.array_equal(t.tags(), before)


def test_find_with_any_subset_of_its_optional_outputs(table):
    t, keys, rows = table
    lib, h, ctx = capi.lib, t.table.handle, t.ctx.handle
    probe = np.concatenate([keys[:8], np.arange(9000, 9008, dtype=np.int64)])      # 8 resident, 8 not
    cached = {int(k): rows[i] for i, k in enumerate(keys)}
    # values and hit mask
    out = np.zeros((probe.size, ROW), np.uint8)
    mask = np.zeros(1, np.uint64)
    assert lib.nve_table_find(h, ctx, probe.size, probe.ctypes.data, mask.ctypes.data, ROW, out.ctypes.data, None) == 0
    t.ctx.wait()
    hits = [(int(mask[0]) >> i) & 1 for i in range(probe.size)]
    assert hits[8:] == [0] * 8 and sum(hits[:8]) > 0
    for i, hit in enumerate(hits):
        if hit:
            assert np.array_equal(out[i], cached[int(probe[i])])
    # only the hit mask
    mask2 = np.zeros(1, np.uint64)
    assert lib.nve_table_find(h, ctx, probe.size, probe.ctypes.data, mask2.ctypes.data, 0, None, None) == 0
    t.ctx.wait()
    assert mask2[0] == mask[0]
    # only the values
    out2 = np.zeros((probe.size, ROW), np.uint8)
    assert lib.nve_table_find(h, ctx, probe.size, probe.ctypes.data, None, ROW, out2.ctypes.data, None) == 0
    t.ctx.wait()
    assert np.array_equal(out2, out)
    # neither: a probe that only moves the miss counter
    t.table.reset_lookup_counter(t.ctx)
    assert lib.nve_table_find(h, ctx, probe.size, probe.ctypes.data, None, 0, None, None) == 0
    t.ctx.wait()
    assert t.table_counter() == probe.size - sum(hits)
    # per-key value sizes are a host-table notion
    sizes = np.zeros(probe.size, np.int64)
    assert lib.nve_table_find(h, ctx, probe.size, probe.ctypes.data, None, ROW, out.ctypes.data,
                              sizes.ctypes.data) != 0


def test_getters_refuse_null_outputs_and_report_the_table(table):
    t, _, _ = table
    lib, h = capi.lib, t.table.handle
    for name in ("nve_table_get_device_id", "nve_table_get_max_row_size", "nve_table_get_key_size"):
        assert getattr(lib, name)(h, None) == INV
    assert lib.nve_table_get_lookup_counter(h, t.ctx.handle, None) == INV
    v32, v64 = C.c_int32(-1), C.c_int64(-1)
    assert lib.nve_table_get_device_id(h, C.byref(v32)) == 0 and v32.value == 0
    assert lib.nve_table_get_max_row_size(h, C.byref(v64)) == 0 and v64.value == ROW
    assert lib.nve_table_get_key_size(h, C.byref(v64)) == 0 and v64.value == 8


def test_lookup_counter_follows_the_misses_after_a_reset(table):
    t, keys, _ = table
    absent = np.arange(50000, 50016, dtype=np.int64)
    assert t.find(absent, None) == 16
    assert t.find(absent[:5], None) == 5          # find() of the helper resets the counter first
    hits = t.find(keys, None)
    assert 0 <= hits < keys.size                   # resident keys do not count
