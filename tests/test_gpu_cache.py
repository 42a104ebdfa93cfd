"""GPU parity of the set-associative cache (probe, hit masks, insert / replacement policy, update,
update_accumulate, erase, clear) through the C ABI against the C oracle: tags per (set, way),
counters, cached bytes, miss counts and looked-up rows must be identical."""
import numpy as np
import pytest

from nv_embedding_cache_b200 import datagen as dg
from nve_helpers import CacheTable
from oracle.pyoracle import OracleCache

pytestmark = pytest.mark.gpu

ROW = 64


def per_set(row=ROW, key_bytes=8):
    return 8 * key_bytes + 8 * row + 32


def table(rows, row=ROW, seed=0):
    t = np.random.default_rng(seed).integers(0, 256, (rows, row), dtype=np.uint8)
    t[:, :8] = np.arange(rows, dtype=np.int64).view(np.uint8).reshape(rows, 8)
    return t


def assert_same_state(gpu: CacheTable, ref: OracleCache, check_counters=True):
    gt, rt = gpu.tags(), ref.tags()
    assert np.array_equal(gt, rt)
    valid = rt != ref.sentinel
    assert np.array_equal(gpu.data()[valid], ref.data()[valid])
    if check_counters:
        assert np.array_equal(gpu.counters()[valid], ref.counters()[valid])


@pytest.mark.parametrize("key_dtype", [np.int32, np.int64])
def test_kats_match_oracle(torch_cuda, oracle, key_dtype):
    kb = np.dtype(key_dtype).itemsize
    t = table(1000)
    gpu = CacheTable(16 * per_set(ROW, kb) + 5, ROW, key_dtype=key_dtype)
    ref = OracleCache(oracle, 16 * per_set(ROW, kb) + 5, ROW, key_dtype)
    assert gpu.num_sets == ref.num_sets == 16
    keys = np.array([5, 9, 1, 999, 7], dtype=key_dtype)
    out = np.full((5, ROW), 0xEE, dtype=np.uint8)
    mask = np.zeros(1, dtype=np.uint64)
    assert gpu.find(keys, out, mask) == 5          # empty cache: every key is a miss
    assert int(mask[0]) == 0 and (out == 0xEE).all()

    ten = np.arange(10, dtype=key_dtype)
    gpu.insert(ten, t[:10])
    ref.insert(ten, values=t[:10])
    assert_same_state(gpu, ref)
    assert sorted(ref.resident_keys().tolist()) == list(range(10))

    probe = np.array(list(range(10)) + [500, 501], dtype=key_dtype)
    for pre in (0, 0b100):
        g_mask, r_mask = np.array([pre], dtype=np.uint64), np.array([pre], dtype=np.uint64)
        g_out, r_out = np.zeros((12, ROW), np.uint8), np.zeros((12, ROW), np.uint8)
        ref.reset_misses()
        ref.lookup(probe, r_out, hit_mask=r_mask)
        assert gpu.find(probe, g_out, g_mask) == ref.misses
        assert np.array_equal(g_mask, r_mask) and np.array_equal(g_out, r_out)

    gpu.erase(np.array([3, 7], dtype=key_dtype))
    ref.invalidate(np.array([3, 7], dtype=key_dtype))
    assert_same_state(gpu, ref)
    g_mask = np.zeros(1, dtype=np.uint64)
    gpu.find(ten, out[:0].reshape(0, ROW) if False else np.zeros((10, ROW), np.uint8), g_mask)
    assert int(g_mask[0]) == 0b1101110111

    gpu.clear()
    ref.clear()
    assert_same_state(gpu, ref)
    assert (gpu.tags() == -1).all()
    gpu.close()


def test_negative_keys(torch_cuda, oracle):
    gpu = CacheTable(13 * per_set(), ROW)
    ref = OracleCache(oracle, 13 * per_set(), ROW)
    keys = np.array([-2, -3, -100, -(1 << 40), 5], dtype=np.int64)
    vals = table(5, seed=3)
    gpu.insert(keys, vals)
    ref.insert(keys, values=vals)
    assert_same_state(gpu, ref)
    out = np.zeros((5, ROW), dtype=np.uint8)
    assert gpu.find(keys, out, np.zeros(1, np.uint64)) == 0
    assert np.array_equal(out, vals)
    gpu.close()


@pytest.mark.parametrize("key_dtype,sets,decay_inserts", [(np.int64, 37, 6), (np.int32, 64, 4), (np.int64, 1, 3)])
def test_random_insert_sequences_match_oracle(torch_cuda, oracle, key_dtype, sets, decay_inserts):
    """Zipf batches with many duplicates into a small cache: sets see far more than 8 candidates,
    equal priorities, hits on resident keys and evictions across inserts."""
    kb = np.dtype(key_dtype).itemsize
    rows = 5000
    t = table(rows, seed=11)
    gpu = CacheTable(sets * per_set(ROW, kb), ROW, key_dtype=key_dtype)
    ref = OracleCache(oracle, sets * per_set(ROW, kb), ROW, key_dtype)
    perm = dg.permutation(rows)
    for step in range(decay_inserts):
        n = [700, 64, 2000, 1, 333, 4096][step]
        keys = dg.zipf_keys(n, rows, 1.2, 100 + step, perm).astype(key_dtype)
        vals = t[keys]
        gpu.insert(keys, vals)
        ref.insert(keys, values=vals)
        assert_same_state(gpu, ref)
        probe = dg.zipf_keys(1000, rows, 1.2, 200 + step, perm).astype(key_dtype)
        g_out, r_out = np.zeros((1000, ROW), np.uint8), np.zeros((1000, ROW), np.uint8)
        g_mask, r_mask = np.zeros(16, np.uint64), np.zeros(16, np.uint64)
        ref.reset_misses()
        ref.lookup(probe, r_out, hit_mask=r_mask)
        assert gpu.find(probe, g_out, g_mask) == ref.misses
        assert np.array_equal(g_mask, r_mask)
        assert np.array_equal(g_out, r_out)
    gpu.close()


def test_max_modify_and_insert_from_backing(torch_cuda, oracle):
    torch = torch_cuda
    rows = 3000
    t = table(rows, seed=5)
    backing = torch.from_numpy(t).cuda()
    gpu = CacheTable(64 * per_set(), ROW, backing=backing, backing_rows=rows, max_modify=50)
    ref = OracleCache(oracle, 64 * per_set(), ROW)
    keys = dg.zipf_keys(1500, rows, 1.05, 9, dg.permutation(rows))
    gpu.insert_from_backing(keys)
    ref.insert(keys, table=t, max_modify=50)
    assert_same_state(gpu, ref)
    assert (ref.tags() != -1).sum() <= 50
    # backed find: every key resolves, misses counted, hit mask untouched by a backed table
    probe = dg.uniform_keys(777, rows, 4)
    out = np.zeros((777, ROW), np.uint8)
    ref.reset_misses()
    r_out = np.zeros_like(out)
    ref.lookup(probe, r_out, table=t)
    assert gpu.find(probe, out) == ref.misses
    assert np.array_equal(out, t[probe]) and np.array_equal(out, r_out)
    gpu.close()


@pytest.mark.parametrize("dtype,npdt", [("f32", np.float32), ("f16", np.float16)])
def test_update_and_accumulate_write_through(torch_cuda, oracle, dtype, npdt):
    torch = torch_cuda
    rows, width = 400, 32
    row_bytes = width * np.dtype(npdt).itemsize
    tf = (np.round(np.random.default_rng(2).normal(size=(rows, width)) * 8) / 8).astype(npdt)
    t = tf.view(np.uint8).reshape(rows, row_bytes)
    backing = torch.from_numpy(t.copy()).cuda()
    gpu = CacheTable(16 * per_set(row_bytes), row_bytes, value_dtype=dtype, backing=backing, backing_rows=rows)
    ref = OracleCache(oracle, 16 * per_set(row_bytes), row_bytes)
    warm = np.arange(0, 120, dtype=np.int64)
    gpu.insert_from_backing(warm)
    ref.insert(warm, table=t)
    keys = np.random.default_rng(3).permutation(rows)[:150].astype(np.int64)   # unique keys
    upd = (np.round(np.random.default_rng(4).normal(size=(150, width)) * 8) / 8).astype(npdt)
    gpu.update_accumulate(keys, upd, dtype)
    ref.update_accumulate(keys, upd)
    host = tf.copy()
    host[keys] = (host[keys].astype(np.float64) + upd.astype(np.float64)).astype(npdt)
    assert_same_state(gpu, ref)
    assert np.array_equal(backing.cpu().numpy(), host.view(np.uint8).reshape(rows, row_bytes))
    new_rows = np.random.default_rng(5).integers(0, 256, (40, row_bytes), dtype=np.uint8)
    gpu.update(keys[:40], new_rows)
    ref.update(keys[:40], new_rows)
    hb = host.view(np.uint8).reshape(rows, row_bytes).copy()
    hb[keys[:40]] = new_rows
    assert_same_state(gpu, ref)
    assert np.array_equal(backing.cpu().numpy(), hb)
    # cache and backing table agree for every key
    out = np.zeros((rows, row_bytes), np.uint8)
    gpu.find(np.arange(rows, dtype=np.int64), out)
    assert np.array_equal(out, hb)
    gpu.close()


def test_two_tier_lookup_with_scatter_merge(torch_cuda, oracle):
    """GPU-tier glue of a multi-tier lookup: the cache serves its hits and reports the hit mask, a
    slower tier (here: the host table, indexed like the batch) resolves every position, and
    nve_b200_scatter_rows merges only the positions the cache missed.  The result is the table's
    rows; hit positions must come from the cache (they are poisoned in the staging buffer)."""
    import ctypes as C
    from nv_embedding_cache_b200 import capi
    from nve_helpers import to_dev
    torch = torch_cuda
    rows, n = 4000, 3000
    t = table(rows, seed=21)
    gpu = CacheTable(64 * per_set(), ROW, key_dtype=np.int64)
    warm = dg.zipf_keys(2000, rows, 1.2, 31, dg.permutation(rows))
    gpu.insert(warm, t[warm])
    keys = dg.zipf_keys(n, rows, 1.2, 32, dg.permutation(rows))
    out = np.zeros((n, ROW), np.uint8)
    mask = np.zeros((n + 63) // 64, np.uint64)
    misses = gpu.find(keys, out, mask)
    bits = ((mask[np.arange(n) // 64] >> (np.arange(n) % 64).astype(np.uint64)) & np.uint64(1)).astype(bool)
    assert 0 < misses < n and int((~bits).sum()) == misses
    staged = t[keys].copy()
    staged[bits] = 0xEE                      # a wrong row wherever the cache already answered
    d_out, d_staged, d_mask = to_dev(torch, out), to_dev(torch, staged), to_dev(torch, mask.view(np.int64))
    capi.check(capi.lib.nve_b200_scatter_rows(d_staged.data_ptr(), ROW, d_out.data_ptr(), ROW, ROW,
                                              d_mask.data_ptr(), n, None))
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy(), t[keys])
    # odd row size and strides: the narrow copy paths
    src = np.random.default_rng(5).integers(0, 256, (50, 23), dtype=np.uint8)
    d_src = to_dev(torch, src)
    d_dst = torch.zeros((50, 29), dtype=torch.uint8, device="cuda")
    capi.check(capi.lib.nve_b200_scatter_rows(d_src.data_ptr(), 23, d_dst.data_ptr(), 29, 21, None, 50, None))
    torch.cuda.synchronize()
    got = d_dst.cpu().numpy()
    assert np.array_equal(got[:, :21], src[:, :21]) and not got[:, 21:].any()
    gpu.close()


@pytest.mark.gpu
def test_host_side_policy_is_the_same_for_both_key_widths(torch_cuda):
    """modify_on_gpu = 0 with int32 and with int64 keys: the same batches leave the same tags (the
    policy works in the key's own width through its unsigned counterpart, like the device probe)."""
    from nve_helpers import CacheTable
    rows, row = 6000, 64
    t = np.random.default_rng(2).integers(0, 256, (rows, row), dtype=np.uint8)
    sets = 41
    c64 = CacheTable(sets * (8 * 8 + 8 * row), row, key_dtype=np.int64, modify_on_gpu=False)
    c32 = CacheTable(sets * (8 * 4 + 8 * row), row, key_dtype=np.int32, modify_on_gpu=False)
    assert c64.num_sets == c32.num_sets == sets
    perm = dg.permutation(rows)
    for step in range(4):
        keys = dg.zipf_keys(1500, rows, 1.15, 40 + step, perm)
        for c in (c64, c32):
            c.insert(keys, t[keys])
        assert np.array_equal(c64.tags(), c32.tags())
        gone = np.unique(keys)[::7]
        for c in (c64, c32):
            c.erase(gone)
        assert np.array_equal(c64.tags(), c32.tags())
        out64, out32 = np.zeros((keys.size, row), np.uint8), np.zeros((keys.size, row), np.uint8)
        m64, m32 = np.zeros((keys.size + 63) // 64, np.uint64), np.zeros((keys.size + 63) // 64, np.uint64)
        c64.find(keys, out64, m64)
        c32.find(keys, out32, m32)
        assert np.array_equal(m64, m32) and np.array_equal(out64, out32)
    c64.close()
    c32.close()
