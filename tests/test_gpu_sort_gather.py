"""The sort-gather schedule of the raw-row lookup against the fused kernel and the table rows.

Both schedules must leave identical bytes in the output (rows of unresolved keys untouched), the
same hit-mask words, the same miss counts and the same set of (position, key) pairs in the miss
list, with and without a cache in front of the backing table."""
import ctypes as C

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import DT, CacheTable, device_read, ptr, to_dev

pytestmark = pytest.mark.gpu


def run_gather(torch, table_dev, rows, row_bytes, keys, *, sorted_tile=None, cache=None, default_row=-1,
               hit_mask=None, miss_list=False, stride=None):
    k_dev = to_dev(torch, keys)
    n = keys.size
    stride = stride or row_bytes
    out = torch.full((n, stride), 0xAB, dtype=torch.uint8, device="cuda")
    g = capi.GatherArgs()
    g.table = ptr(table_dev) if table_dev is not None else None
    g.num_rows = rows
    g.row_stride = row_bytes
    g.value_dtype = DT["f16"]
    g.default_row_index = default_row
    g.cache = C.pointer(cache) if cache is not None else None
    g.key_type = capi.KEY_INT64 if keys.dtype == np.int64 else capi.KEY_INT32
    g.keys = ptr(k_dev)
    g.num_keys = n
    g.output = ptr(out)
    g.output_stride = stride
    g.output_dtype = DT["f16"]
    g.row_copy_bytes = row_bytes
    mask_dev = None
    if hit_mask is not None:
        mask_dev = to_dev(torch, hit_mask)
        g.hit_mask = ptr(mask_dev)
    miss = torch.zeros(1, dtype=torch.int64, device="cuda")
    g.miss_count = ptr(miss)
    pos = mkeys = cursor = None
    if miss_list:
        pos = torch.full((n,), -7, dtype=torch.int64, device="cuda")
        mkeys = torch.full((n,), -7, dtype=torch.int64 if keys.dtype == np.int64 else torch.int32, device="cuda")
        cursor = torch.zeros(1, dtype=torch.int64, device="cuda")
        g.miss_positions, g.miss_keys, g.miss_list_len = ptr(pos), ptr(mkeys), ptr(cursor)
    if sorted_tile is None:
        capi.check(capi.lib.nve_b200_gather_rows(C.byref(g), None))
    else:
        need = C.c_size_t(0)
        capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), sorted_tile, None, C.byref(need), None))
        scratch = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
        capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), sorted_tile, ptr(scratch), C.byref(need), None))
    torch.cuda.synchronize()
    res = {"out": out.cpu().numpy(), "miss": int(miss.item()),
           "mask": None if mask_dev is None else mask_dev.cpu().numpy()}
    if miss_list:
        m = int(cursor.item())
        res["miss_list"] = sorted(zip(pos[:m].cpu().tolist(), mkeys[:m].cpu().tolist()))
    return res


def same(a, b):
    assert np.array_equal(a["out"], b["out"])
    assert a["miss"] == b["miss"]
    if a["mask"] is not None:
        assert np.array_equal(a["mask"], b["mask"])
    if "miss_list" in a:
        assert a["miss_list"] == b["miss_list"]


@pytest.mark.parametrize("row_bytes", [2, 6, 20, 64, 130, 256, 512, 1028, 4096])
@pytest.mark.parametrize("key_dtype", [np.int32, np.int64])
def test_table_only_row_sizes(torch_cuda, row_bytes, key_dtype):
    """No cache: every vector width and lane-group width of the copy kernel, ragged batch."""
    torch = torch_cuda
    rows = 700
    table = np.random.default_rng(row_bytes).integers(0, 256, (rows, row_bytes), dtype=np.uint8)
    keys = dg.uniform_keys(1237, rows, 3).astype(key_dtype)
    t_dev = to_dev(torch, table)
    got = run_gather(torch, t_dev, rows, row_bytes, keys, sorted_tile=0)
    assert np.array_equal(got["out"], table[keys])
    assert got["miss"] == 0


def test_tiles_of_several_groups(torch_cuda):
    """A batch large enough that a warp's tile spans several groups of 32 sorted words."""
    torch = torch_cuda
    rows, rb, n = 70000, 64, 400_003
    table = np.random.default_rng(2).integers(0, 256, (rows, rb), dtype=np.uint8)
    keys = dg.uniform_keys(n, rows, 4)
    keys[::1001] = -1                                   # unresolved: sorted last, rows untouched
    got = run_gather(torch, to_dev(torch, table), rows, rb, keys, sorted_tile=4096)
    want = table[np.where(keys < 0, 0, keys)]
    want[keys < 0] = 0xAB
    assert np.array_equal(got["out"], want)
    assert got["miss"] == int((keys < 0).sum())


@pytest.mark.parametrize("tile", [0, 32, 100, 4096])
def test_unresolved_keys_default_row_and_masks(torch_cuda, tile):
    torch = torch_cuda
    rows, rb, n = 300, 64, 1000
    table = np.random.default_rng(1).integers(0, 256, (rows, rb), dtype=np.uint8)
    t_dev = to_dev(torch, table)
    keys = dg.uniform_keys(n, rows, 2)
    keys[[3, 64, 65, 200, 332, 999]] = [-5, rows, 1 << 40, -1, 999, rows + 1]
    mask = np.zeros((n + 63) // 64, dtype=np.uint64)
    for i in (0, 31, 32, 63, 64, 100, 331, 998):
        mask[i // 64] |= np.uint64(1) << np.uint64(i % 64)
    for default_row in (-1, 17):
        a = run_gather(torch, t_dev, rows, rb, keys, hit_mask=mask.copy(), miss_list=True,
                       default_row=default_row, stride=96)
        b = run_gather(torch, t_dev, rows, rb, keys, hit_mask=mask.copy(), miss_list=True,
                       default_row=default_row, stride=96, sorted_tile=tile)
        same(a, b)
        assert (a["miss"] == 5) == (default_row < 0)
        assert np.all(b["out"][:, rb:] == 0xAB)          # padding of the output rows stays untouched


@pytest.mark.parametrize("key_dtype", [np.int64, np.int32])
@pytest.mark.parametrize("host_table", [False, True])
def test_cache_in_front_of_table(torch_cuda, key_dtype, host_table):
    """A populated cache in front of a device or pinned-host table: rows come from both, the miss
    counter of the cache and the outputs agree with the fused kernel; cache-only lookups (no table)
    leave the rows of missing keys untouched."""
    torch = torch_cuda
    rows, rb, n = 20000, 256, 50001
    table = np.random.default_rng(5).integers(0, 256, (rows, rb), dtype=np.uint8)
    backing = torch.from_numpy(table).pin_memory() if host_table else to_dev(torch, table)
    ct = CacheTable(64 * (8 * np.dtype(key_dtype).itemsize + 8 * rb + 32), rb, key_dtype=key_dtype,
                    backing=backing, backing_rows=rows)
    warm = dg.zipf_keys(4000, rows, 1.1, 7, dg.permutation(rows))
    ct.insert(warm, table[warm])
    keys = dg.zipf_keys(n, rows, 1.1, 8, dg.permutation(rows)).astype(key_dtype)

    def misses():
        return int(device_read(ct.view.misses, 8).view(np.int64)[0])

    m0 = misses()
    a = run_gather(torch, backing, rows, rb, keys, cache=ct.view)
    m1 = misses()
    b = run_gather(torch, backing, rows, rb, keys, cache=ct.view, sorted_tile=0)
    m2 = misses()
    same(a, b)
    assert np.array_equal(b["out"], table[keys])
    assert 0 < m1 - m0 == m2 - m1 < n
    a = run_gather(torch, None, 0, rb, keys, cache=ct.view, miss_list=True)
    b = run_gather(torch, None, 0, rb, keys, cache=ct.view, miss_list=True, sorted_tile=64)
    same(a, b)
    assert a["miss"] == m1 - m0
    ct.close()


def test_table_schedule_selection(torch_cuda):
    """GpuTable.find with kernel_mode_type 2 (sort-gather, tile from kernel_mode_value), with the
    dynamic mode's threshold and with type 3 (pipeline: host threads gather the table rows) returns
    what the fused schedule (mode 1) returns."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GpuTable
    rows, rb, n = 30000, 128, 40000
    table = np.random.default_rng(9).integers(0, 256, (rows, rb), dtype=np.uint8)
    backing = torch.from_numpy(table).pin_memory()
    keys = dg.zipf_keys(n, rows, 1.05, 3, dg.permutation(rows))
    warm = dg.zipf_keys(5000, rows, 1.05, 4, dg.permutation(rows))
    outs, counters = [], []
    class PipelineParams(C.Structure):
        _fields_ = [("task_size", C.c_uint64), ("num_aux_streams", C.c_uint64)]
    small_tasks = PipelineParams(100, 3)
    one_stream = PipelineParams(0, 0)
    for mode, value in ((1, 0), (2, 0), (2, 256), (0, 1000), (0, 0), (3, 0),
                        (3, C.addressof(small_tasks)), (3, C.addressof(one_stream))):
        gt = GpuTable(128 * (64 + 8 * rb + 32), rb, "float16", uvm_table=backing, uvm_num_rows=rows,
                      kernel_mode_type=mode, kernel_mode_value=value)
        ctx = gt.create_execution_context()
        gt.insert(ctx, warm.size, warm, rb, rb, table[warm])
        ctx.wait()
        out = np.zeros((n, rb), np.uint8)
        gt.reset_lookup_counter(ctx)
        gt.find(ctx, n, keys, None, rb, out)
        ctx.wait()
        v = C.c_int64(-1)
        capi.check(capi.lib.nve_table_get_lookup_counter(gt.handle, ctx.handle, C.byref(v)))
        ctx.wait()
        outs.append(out)
        counters.append(v.value)
        ctx.destroy()
        gt.destroy()
    for o in outs:
        assert np.array_equal(o, table[keys])
    assert len(set(counters)) == 1 and 0 < counters[0] < n


def test_pipeline_schedule_repeated_and_device_table(torch_cuda):
    """The pipeline schedule over several lookups with inserts between them (staging buffers are
    reused, the cache changes), with no misses at all, and on a table in device memory, where host
    threads cannot read the rows and the lookup takes the fused kernel instead."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GpuTable
    rows, rb = 5000, 64
    table = np.random.default_rng(19).integers(0, 256, (rows, rb), dtype=np.uint8)
    for backing in (torch.from_numpy(table).pin_memory(), to_dev(torch, table)):
        gt = GpuTable(512 * (64 + 8 * rb + 32), rb, "float16", uvm_table=backing, uvm_num_rows=rows,
                      kernel_mode_type=3)
        ctx = gt.create_execution_context()
        for step in range(4):
            n = 3000 + 517 * step
            keys = dg.zipf_keys(n, rows, 1.1, 30 + step, dg.permutation(rows))
            out = np.zeros((n, rb), np.uint8)
            gt.find(ctx, n, keys, None, rb, out)
            ctx.wait()
            assert np.array_equal(out, table[keys])
            gt.insert(ctx, n, keys, rb, rb, table[keys])
            ctx.wait()
        hot = np.repeat(keys[:8], 50)                   # every key resident: nothing for the host half
        out = np.zeros((hot.size, rb), np.uint8)
        gt.reset_lookup_counter(ctx)
        gt.find(ctx, hot.size, hot, None, rb, out)
        ctx.wait()
        assert np.array_equal(out, table[hot])
        ctx.destroy()
        gt.destroy()


def test_pipeline_schedule_with_a_thread_pool_of_the_callers(torch_cuda):
    """An execution context created with a pool from nve_thread_pool_create stages its table rows
    on that pool's threads (one worker, then five); outputs are those of the default pool.  The pool
    handle may be destroyed while a context still uses it.  Once the default pool has served a
    lookup it can no longer be re-sized (the reference refuses the same,
    tests/c_api/c_api_threadpool_test.cpp:72-104)."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import ExecutionContext, GpuTable
    rows, rb = 6000, 128
    table = np.random.default_rng(23).integers(0, 256, (rows, rb), dtype=np.uint8)
    backing = torch.from_numpy(table).pin_memory()
    gt = GpuTable(256 * (64 + 8 * rb + 32), rb, "float16", uvm_table=backing, uvm_num_rows=rows, kernel_mode_type=3)
    keys = dg.zipf_keys(20000, rows, 1.05, 77, dg.permutation(rows))
    default_ctx = gt.create_execution_context()
    want = np.zeros((keys.size, rb), np.uint8)
    gt.find(default_ctx, keys.size, keys, None, rb, want)
    default_ctx.wait()
    assert np.array_equal(want, table[keys])
    for workers in (1, 5):
        pool = C.c_void_p()
        capi.check(capi.lib.nve_thread_pool_create(C.byref(pool), b'{"name": "simple", "num_workers": %d}' % workers))
        h = C.c_void_p()
        capi.check(capi.lib.nve_table_create_execution_context(gt.handle, C.byref(h), None, None, pool, None))
        capi.check(capi.lib.nve_thread_pool_destroy(pool))          # the context keeps the threads
        ctx = ExecutionContext(h)
        out = np.zeros((keys.size, rb), np.uint8)
        gt.find(ctx, keys.size, keys, None, rb, out)
        ctx.wait()
        assert np.array_equal(out, want)
        ctx.destroy()
    assert capi.lib.nve_configure_default_thread_pool(b'{"name": "simple", "num_workers": 2}') == capi.NVE_ERROR_RUNTIME
    assert "already in use" in capi.last_error()
    default_ctx.destroy()
    gt.destroy()


def test_rejections(torch_cuda):
    torch = torch_cuda
    table = np.zeros((10, 64), np.uint8)
    t_dev = to_dev(torch, table)
    keys = to_dev(torch, np.arange(10, dtype=np.int64))
    out = torch.zeros((10, 32), dtype=torch.float32, device="cuda")
    g = capi.GatherArgs()
    g.table, g.num_rows, g.row_stride, g.value_dtype, g.row_width = ptr(t_dev), 10, 64, DT["f16"], 32
    g.default_row_index, g.key_type, g.keys, g.num_keys = -1, capi.KEY_INT64, ptr(keys), 10
    g.output, g.output_stride, g.output_dtype = ptr(out), 128, DT["f32"]     # a decoding lookup
    need = C.c_size_t(0)
    with pytest.raises(capi.NveError) as e:
        capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), 0, None, C.byref(need), None))
    assert e.value.status == capi.NVE_ERROR_INVALID_ARGUMENT
    g.output_dtype, g.row_copy_bytes, g.output_stride = DT["f16"], 64, 64
    capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), 0, None, C.byref(need), None))
    assert need.value > 0
    small = C.c_size_t(need.value - 1)
    scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.NveError):
        capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), 0, ptr(scratch), C.byref(small), None))
    with pytest.raises(capi.NveError):
        capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), 0, None, None, None))
