"""This library against the UNMODIFIED reference GPU code on the same GPU (and the C oracle against
both): the set-associative cache with its device-side replacement policy, the Deduper, the
gradient de-duplication and the pooled find_and_combine kernel.

Integer state (tags per (set, way), hit masks, miss counts, unique keys, counts, offsets, inverse
positions, chunk maps) and copied rows must be identical.  Floating-point sums must agree exactly
where the reference adds in a fixed order and within 1e-5 relative (1e-6 for gradient sums) where
it uses atomics or fused multiply-adds.  The cache is compared under both of its modify policies:
decided on the device (the default) and decided on the host (modify_on_gpu = 0)."""
import ctypes as C

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import CacheTable, GpuLayer, device_read, to_dev
from oracle.pyoracle import OracleCache, RefGpuDeduper

pytestmark = pytest.mark.gpu

ROW = 64


def per_set(row=ROW, key_bytes=8):
    return 8 * key_bytes + 8 * row + 32


def byte_table(rows, row=ROW, seed=0):
    t = np.random.default_rng(seed).integers(0, 256, (rows, row), dtype=np.uint8)
    t[:, :8] = np.arange(rows, dtype=np.int64).view(np.uint8).reshape(rows, 8)
    return t


def ref_tags(cache):
    n, tags, _ = cache.view()
    return device_read(tags, n * 8 * 8).view(np.int64).reshape(n, 8)


def ref_rows(cache, row_bytes):
    n, _, rows = cache.view()
    return device_read(rows, n * 8 * row_bytes).reshape(n, 8, row_bytes)


@pytest.mark.parametrize("sets,steps", [(37, 6), (1, 3), (256, 6)])
def test_cache_state_after_inserts(torch_cuda, oracle, reference_gpu, sets, steps):
    """Zipf batches with many duplicates into a small cache (sets see more than 8 candidates, equal
    priorities, resident keys hit again, evictions across inserts): after every insert the tags of
    every (set, way), the cached rows, hit masks, miss counts and looked-up rows are the same in
    the reference cache, this library's cache and the C oracle."""
    torch = torch_cuda
    rows = 5000
    t = byte_table(rows, seed=11)
    t_dev = to_dev(torch, t)
    cache_bytes = sets * per_set()
    mine = CacheTable(cache_bytes, ROW, key_dtype=np.int64)
    orc = OracleCache(oracle, cache_bytes, ROW, np.int64)
    ref = reference_gpu.cache(cache_bytes, ROW)
    assert ref.view()[0] == mine.num_sets == sets
    perm = dg.permutation(rows)
    for step in range(steps):
        n = [700, 64, 2000, 1, 333, 4096][step]
        keys = dg.zipf_keys(n, rows, 1.2, 100 + step, perm)
        vals = t[keys]
        k_dev, v_dev = to_dev(torch, keys), to_dev(torch, vals)
        mine.insert(keys, vals)
        orc.insert(keys, values=vals)
        ref.insert(k_dev.data_ptr(), n, v_dev.data_ptr(), ROW)
        rt = ref_tags(ref)
        assert np.array_equal(orc.tags(), rt), f"oracle vs reference tags, insert {step}"
        assert np.array_equal(mine.tags(), rt), f"library vs reference tags, insert {step}"
        valid = rt != -1
        assert np.array_equal(mine.data()[valid], ref_rows(ref, ROW)[valid])

        probe = dg.zipf_keys(1000, rows, 1.2, 200 + step, perm)
        p_dev = to_dev(torch, probe)
        r_out = torch.zeros((1000, ROW), dtype=torch.uint8, device="cuda")
        r_mask = torch.zeros(16, dtype=torch.int64, device="cuda")
        r_miss = ref.lookup_mask(p_dev.data_ptr(), 1000, r_out.data_ptr(), ROW, r_mask.data_ptr())
        g_out, g_mask = np.zeros((1000, ROW), np.uint8), np.zeros(16, np.uint64)
        g_miss = mine.find(probe, g_out, g_mask)
        assert g_miss == r_miss
        assert np.array_equal(g_mask, r_mask.cpu().numpy().view(np.uint64))
        assert np.array_equal(g_out, r_out.cpu().numpy())
        # table-backed lookup: every row resolved, from the cache or from the table
        r_out.zero_()
        ref.lookup_table(p_dev.data_ptr(), 1000, r_out.data_ptr(), ROW, t_dev.data_ptr())
        assert np.array_equal(r_out.cpu().numpy(), t[probe])
    mine.close()
    ref.close()


def test_cache_modify_ops(torch_cuda, oracle, reference_gpu):
    """update, update_accumulate (fp32), invalidate and clear leave the same tags and rows."""
    torch = torch_cuda
    rows, width = 3000, 16                       # 16 fp32 values = 64-byte rows
    t = dg.dyadic_table(rows, width, 3, np.float32)
    cache_bytes = 64 * per_set()
    mine = CacheTable(cache_bytes, ROW, value_dtype="f32", key_dtype=np.int64)
    ref = reference_gpu.cache(cache_bytes, ROW)
    keys = dg.zipf_keys(1500, rows, 1.1, 7, dg.permutation(rows))
    vals = t[keys].view(np.uint8).reshape(-1, ROW)
    mine.insert(keys, vals)
    k_dev, v_dev = to_dev(torch, keys), to_dev(torch, vals)     # named: they must outlive the call
    ref.insert(k_dev.data_ptr(), keys.size, v_dev.data_ptr(), ROW)
    assert np.array_equal(mine.tags(), ref_tags(ref))

    uk = np.unique(keys)[:400]
    new = dg.dyadic_table(uk.size, width, 31, np.float32)
    mine.update(uk, new.view(np.uint8).reshape(-1, ROW))
    uk_dev, new_dev = to_dev(torch, uk), to_dev(torch, new)
    ref.update(uk_dev.data_ptr(), uk.size, new_dev.data_ptr(), ROW)
    valid = ref_tags(ref) != -1
    assert np.array_equal(mine.data()[valid], ref_rows(ref, ROW)[valid])

    upd = dg.dyadic_table(uk.size, width, 32, np.float32)
    mine.update_accumulate(uk, upd, "f32")
    upd_dev = to_dev(torch, upd)
    ref.update_accumulate(uk_dev.data_ptr(), uk.size, upd_dev.data_ptr(), ROW)
    assert np.array_equal(mine.data()[valid], ref_rows(ref, ROW)[valid])

    gone = np.unique(keys)[100:300]
    mine.erase(gone)
    gone_dev = to_dev(torch, gone)
    ref.invalidate(gone_dev.data_ptr(), gone.size)
    assert np.array_equal(mine.tags(), ref_tags(ref))
    mine.clear()
    ref.clear()
    assert np.array_equal(mine.tags(), ref_tags(ref))
    assert (mine.tags() == -1).all()
    mine.close()
    ref.close()


class MyDeduper:
    def __init__(self, max_run, n):
        self.h = C.c_void_p()
        capi.check(capi.lib.nve_b200_deduper_create(C.byref(self.h), capi.KEY_INT64, max_run, n))

    def close(self):
        capi.check(capi.lib.nve_b200_deduper_destroy(self.h))


def dedup_buffers(torch, n, max_run):
    cap = n + (n // max_run if max_run > 0 else 0) + 2
    mk = lambda m: torch.full((m,), -7, dtype=torch.int64, device="cuda")
    return dict(unique=mk(n + 1), counts=mk(n + 1), inverse=mk(n + 1), offsets=mk(cap + 1), loc_map=mk(cap + 1))


@pytest.mark.parametrize("max_run", [-1, 8, 1024])
@pytest.mark.parametrize("end_bit", [0, 13])
def test_deduper_outputs(torch_cuda, oracle, reference_gpu, max_run, end_bit):
    torch = torch_cuda
    n, rows = 50000, 6000
    keys = dg.zipf_keys(n, rows, 1.05, 21, dg.permutation(rows))
    keys[::5] = keys[3]
    k_dev = to_dev(torch, keys)
    a, b = dedup_buffers(torch, n, max_run), dedup_buffers(torch, n, max_run)
    rd = RefGpuDeduper(reference_gpu, max_run, n)
    ru, rc = rd.dedup(k_dev.data_ptr(), n, b["unique"].data_ptr(), b["counts"].data_ptr(),
                      b["loc_map"].data_ptr(), b["inverse"].data_ptr(), b["offsets"].data_ptr(), end_bit)
    md = MyDeduper(max_run, n)
    runs = np.zeros(2, np.int64)
    capi.check(capi.lib.nve_b200_deduper_dedup(md.h, k_dev.data_ptr(), n, a["unique"].data_ptr(),
                                               a["counts"].data_ptr(), a["loc_map"].data_ptr(),
                                               runs.ctypes.data, a["inverse"].data_ptr(),
                                               a["offsets"].data_ptr(), None, end_bit))
    assert (int(runs[0]), int(runs[1])) == (ru, rc)
    o = oracle.dedup(keys, max_run=max_run, end_bit=end_bit)
    assert (o["num_unique"], o["num_chunks"]) == (ru, rc)
    for name, m in (("unique", ru), ("counts", ru), ("inverse", n), ("offsets", rc + 1)):
        ref_arr = b[name][:m].cpu().numpy()
        assert np.array_equal(a[name][:m].cpu().numpy(), ref_arr), name
        assert np.array_equal(o[name], ref_arr), "oracle " + name
    if max_run > 0:
        ref_arr = b["loc_map"][:rc].cpu().numpy()
        assert np.array_equal(a["loc_map"][:rc].cpu().numpy(), ref_arr)
        assert np.array_equal(o["loc_map"], ref_arr)
    md.close()
    rd.close()


@pytest.mark.parametrize("max_run", [-1, 1024])
@pytest.mark.parametrize("width", [32, 128])
def test_gradient_sums(torch_cuda, reference_gpu, max_run, width):
    """Per-key gradient sums.  The reference adds the rows of a chunk in position order, so
    un-split groups are bit-identical; split groups are combined with atomics there (any order) and
    in chunk order here, hence a tolerance for those and exact equality on dyadic data."""
    torch = torch_cuda
    n, rows = 40000, 3000
    keys = dg.zipf_keys(n, rows, 1.05, 5, dg.permutation(rows))
    keys[::4] = keys[0]                      # one group far longer than 1024
    k_dev = to_dev(torch, keys)
    b = dedup_buffers(torch, n, max_run)
    rd = RefGpuDeduper(reference_gpu, max_run, n)
    u, c = rd.dedup(k_dev.data_ptr(), n, b["unique"].data_ptr(), b["counts"].data_ptr(),
                    b["loc_map"].data_ptr(), b["inverse"].data_ptr(), b["offsets"].data_ptr())
    md = MyDeduper(max_run, n)
    a = dedup_buffers(torch, n, max_run)
    runs = np.zeros(2, np.int64)
    capi.check(capi.lib.nve_b200_deduper_dedup(md.h, k_dev.data_ptr(), n, a["unique"].data_ptr(),
                                               a["counts"].data_ptr(), a["loc_map"].data_ptr(),
                                               runs.ctypes.data, a["inverse"].data_ptr(),
                                               a["offsets"].data_ptr(), None, 0))
    for grads_np, exact in ((dg.dyadic_table(n, width, 6, np.float32), True),
                            (np.random.default_rng(7).normal(0, 1e-2, (n, width)).astype(np.float32), False)):
        g = to_dev(torch, grads_np)
        want = torch.zeros((u, width), device="cuda")
        rd.grads(g.data_ptr(), want.data_ptr(), b["unique"].data_ptr(), b["inverse"].data_ptr(),
                 b["loc_map"].data_ptr() if max_run > 0 else None, b["offsets"].data_ptr(), u, c, width)
        got = torch.full((u, width), 5.0, device="cuda")
        capi.check(capi.lib.nve_b200_dedup_grads(md.h, g.data_ptr(), width * 4, width * 4, n,
                                                 a["unique"].data_ptr(), a["inverse"].data_ptr(),
                                                 a["offsets"].data_ptr(), a["loc_map"].data_ptr(),
                                                 got.data_ptr(), width * 4, 0, 0, 1.0, None))
        torch.cuda.synchronize()
        got_np, want_np = got.cpu().numpy(), want.cpu().numpy()
        if exact or max_run == -1:
            assert np.array_equal(got_np, want_np)
        else:
            scale = max(1.0, float(np.abs(want_np).max()))
            assert np.max(np.abs(got_np - want_np)) <= 1e-6 * scale * 4
            counts = b["counts"][:u].cpu().numpy()
            short = counts <= 1024             # groups of a single chunk: same order of additions
            assert np.array_equal(got_np[short], want_np[short])
    md.close()
    rd.close()


@pytest.mark.parametrize("width", [128, 32, 20])
def test_update_accumulate_table(torch_cuda, reference_gpu, width):
    """table[key] += row against the reference's UpdateAccumulateTable: with unique keys each table
    element takes exactly one fp32 addition, so both paths (atomic and load/store) are bit-identical;
    keys outside the table are skipped by both."""
    torch = torch_cuda
    rows, n = 5000, 1500
    rng = np.random.default_rng(11)
    keys = rng.permutation(rows)[:n].astype(np.int64)
    keys[::97] = rows + 5                      # out of range: skipped
    keys[5] = -3
    table_np = rng.normal(0, 1, (rows, width)).astype(np.float32)
    upd = to_dev(torch, rng.normal(0, 1e-2, (n, width)).astype(np.float32))
    k_dev = to_dev(torch, keys)
    want = to_dev(torch, table_np)
    reference_gpu.update_accumulate_table(upd.data_ptr(), k_dev.data_ptr(), want.data_ptr(), width, n, rows)
    for unique in (0, 1):
        got = to_dev(torch, table_np)
        capi.check(capi.lib.nve_b200_update_rows(got.data_ptr(), rows, width * 4, capi.DTYPE_FLOAT32, width * 4,
                                                 capi.KEY_INT64, k_dev.data_ptr(), n, upd.data_ptr(), width * 4,
                                                 1, unique, None))
        torch.cuda.synchronize()
        assert torch.equal(got, want)


@pytest.mark.parametrize("max_run", [-1, 1024])
def test_gradient_sums_fp16(torch_cuda, reference_gpu, max_run):
    """fp16 gradient rows are added in fp16, in position order: un-split groups are bit-identical to
    the reference kernel and to a one-rounding-per-addition evaluation on the host; split groups
    (half atomics in the reference, any order) within fp16 accumulation error."""
    torch = torch_cuda
    n, rows, width = 30000, 2500, 64
    keys = dg.zipf_keys(n, rows, 1.05, 15, dg.permutation(rows))
    keys[::4] = keys[0]
    k_dev = to_dev(torch, keys)
    b = dedup_buffers(torch, n, max_run)
    rd = RefGpuDeduper(reference_gpu, max_run, n)
    u, c = rd.dedup(k_dev.data_ptr(), n, b["unique"].data_ptr(), b["counts"].data_ptr(),
                    b["loc_map"].data_ptr(), b["inverse"].data_ptr(), b["offsets"].data_ptr())
    md = MyDeduper(max_run, n)
    a = dedup_buffers(torch, n, max_run)
    runs = np.zeros(2, np.int64)
    capi.check(capi.lib.nve_b200_deduper_dedup(md.h, k_dev.data_ptr(), n, a["unique"].data_ptr(),
                                               a["counts"].data_ptr(), a["loc_map"].data_ptr(),
                                               runs.ctypes.data, a["inverse"].data_ptr(),
                                               a["offsets"].data_ptr(), None, 0))
    grads_np = np.random.default_rng(3).normal(0, 0.05, (n, width)).astype(np.float16)
    g = to_dev(torch, grads_np)
    want = torch.zeros((u, width), dtype=torch.float16, device="cuda")
    rd.grads_f16(g.data_ptr(), want.data_ptr(), b["unique"].data_ptr(), b["inverse"].data_ptr(),
                 b["loc_map"].data_ptr() if max_run > 0 else None, b["offsets"].data_ptr(), u, c, width)
    got = torch.full((u, width), 5.0, dtype=torch.float16, device="cuda")
    capi.check(capi.lib.nve_b200_dedup_grads_f16(md.h, g.data_ptr(), width * 2, width * 2, n,
                                                 a["inverse"].data_ptr(), a["offsets"].data_ptr(),
                                                 a["loc_map"].data_ptr(), got.data_ptr(), width * 2, None))
    torch.cuda.synchronize()
    got_np, want_np = got.cpu().numpy(), want.cpu().numpy()
    counts = b["counts"][:u].cpu().numpy()
    short = counts <= 1024 if max_run > 0 else np.ones(u, bool)
    assert np.array_equal(got_np[short], want_np[short])
    assert np.max(np.abs(got_np.astype(np.float32) - want_np.astype(np.float32))) <= 0.25
    # host evaluation, one fp16 rounding per addition, for a sample of short groups
    inv, offs = a["inverse"][:n].cpu().numpy(), a["offsets"][:c + 1].cpu().numpy()
    if max_run == -1:
        for grp in list(range(0, u, max(1, u // 40)))[:40]:
            acc = np.zeros(width, np.float16)
            for pos in inv[offs[grp]:offs[grp + 1]]:
                acc = (acc.astype(np.float64) + grads_np[pos].astype(np.float64)).astype(np.float16)
            assert np.array_equal(acc, got_np[grp]), grp
    md.close()
    rd.close()


def test_pooled_lookup_fp16(torch_cuda, reference_gpu):
    """fp16 rows: CSR bags with mean pooling and fixed-hotness sum pooling against the reference's
    find_and_combine kernel reading the table directly."""
    torch = torch_cuda
    rows, width, bags = 20000, 128, 3000
    t = dg.normal_table(rows, width, 0.02, 3, np.float16)
    t_dev = to_dev(torch, t)
    lens = np.random.default_rng(4).integers(1, 33, bags)
    offs = np.zeros(bags + 1, np.int64)
    offs[1:] = np.cumsum(lens)
    keys = dg.zipf_keys(int(offs[-1]), rows, 1.1, 5, dg.permutation(rows))
    k_dev, o_dev = to_dev(torch, keys), to_dev(torch, offs)
    layer = GpuLayer(t_dev, rows, width * 2, "f16")
    want = torch.zeros((bags, width), dtype=torch.float16, device="cuda")
    reference_gpu.find_and_combine("f16_csr_mean", bags, t_dev.data_ptr(), [k_dev.data_ptr()],
                                   [o_dev.data_ptr()], 0, width, want.data_ptr())
    got = torch.zeros_like(want)
    layer.lookup_pooled(k_dev, got, width * 2, "mean", offsets=o_dev, out_dtype="f16")
    layer.ctx.wait()
    g, w = got.cpu().numpy().astype(np.float32), want.cpu().numpy().astype(np.float32)
    assert np.max(np.abs(g - w)) <= np.maximum(np.abs(w), 2.0 ** -14).max() * 2.0 ** -10   # one fp16 ulp
    assert np.mean(g == w) > 0.99

    hot = 8
    keys2 = keys[: bags * hot]
    k2 = to_dev(torch, keys2)
    reference_gpu.find_and_combine("f16_fixed_sum", bags, t_dev.data_ptr(), [k2.data_ptr()], None, hot,
                                   width, want.data_ptr())
    layer.lookup_pooled(k2, got, width * 2, "sum", hotness=hot, out_dtype="f16")
    layer.ctx.wait()
    g, w = got.cpu().numpy().astype(np.float32), want.cpu().numpy().astype(np.float32)
    assert np.max(np.abs(g - w)) <= np.maximum(np.abs(w), 2.0 ** -14).max() * 2.0 ** -10
    assert np.mean(g == w) > 0.99
    layer.close()


def test_pooled_lookup_int8(torch_cuda, reference_gpu):
    """int8 rows with an fp32 row scale, tight 260-byte rows, fixed hotness, sum -> fp32."""
    torch = torch_cuda
    rows, width, bags, hot = 20000, 256, 2000, 20
    t = dg.quantized_rows(rows, width, 9, "qint8_f32")
    assert t.shape[1] == 260
    t_dev = to_dev(torch, t)
    keys = dg.zipf_keys(bags * hot, rows, 1.05, 6, dg.permutation(rows))
    k_dev = to_dev(torch, keys)
    want = torch.zeros((bags, width), dtype=torch.float32, device="cuda")
    reference_gpu.find_and_combine("qint8_fixed_sum", bags, t_dev.data_ptr(), [k_dev.data_ptr()], None, hot,
                                   width, want.data_ptr())
    layer = GpuLayer(t_dev, rows, 260, "qint8_f32")
    got = torch.zeros_like(want)
    layer.lookup_pooled(k_dev, got, width * 4, "sum", hotness=hot, out_dtype="f32")
    layer.ctx.wait()
    g, w = got.cpu().numpy(), want.cpu().numpy()
    assert np.max(np.abs(g - w) / np.maximum(np.abs(w), 1e-3)) <= 1e-5
    layer.close()


# ---- the host-side modify policy (modify_on_gpu = 0) --------------------------------------------
def per_set_host(row=ROW, key_bytes=8):
    """Bytes of cache_size one set takes when the counters live on the host."""
    return 8 * key_bytes + 8 * row


@pytest.mark.parametrize("sets,steps", [(37, 6), (1, 3), (256, 6)])
def test_host_policy_cache_state_after_inserts(torch_cuda, reference_gpu, sets, steps):
    """The same Zipf batches as for the device policy, through the reference's CacheSAHostModify (fed
    by its host histogram) and through this library's table with modify_on_gpu = 0: the policy is
    sequential and deterministic, so the tags of every (set, way), the cached rows, hit masks and
    looked-up rows must be identical after every insert."""
    torch = torch_cuda
    rows = 5000
    t = byte_table(rows, seed=11)
    cache_bytes = sets * per_set_host()
    mine = CacheTable(cache_bytes, ROW, key_dtype=np.int64, modify_on_gpu=False)
    ref = reference_gpu.host_cache(cache_bytes, ROW)
    assert ref.view()[0] == mine.num_sets == sets
    perm = dg.permutation(rows)
    for step in range(steps):
        n = [700, 64, 2000, 1, 333, 4096][step]
        keys = dg.zipf_keys(n, rows, 1.2, 100 + step, perm)
        vals = t[keys]
        v_dev = to_dev(torch, vals)
        mine.insert(keys, vals)
        ref.insert(keys.ctypes.data, n, v_dev.data_ptr(), ROW)
        rt = ref_tags(ref)
        assert np.array_equal(mine.tags(), rt), f"library vs reference tags, insert {step}"
        valid = rt != -1
        assert valid.any()
        assert np.array_equal(mine.data()[valid], ref_rows(ref, ROW)[valid])

        probe = dg.zipf_keys(1000, rows, 1.2, 200 + step, perm)
        p_dev = to_dev(torch, probe)
        r_out = torch.zeros((1000, ROW), dtype=torch.uint8, device="cuda")
        r_mask = torch.zeros(16, dtype=torch.int64, device="cuda")
        ref.lookup_mask(p_dev.data_ptr(), 1000, r_out.data_ptr(), ROW, r_mask.data_ptr())
        g_out, g_mask = np.zeros((1000, ROW), np.uint8), np.zeros(16, np.uint64)
        mine.find(probe, g_out, g_mask)
        assert np.array_equal(g_mask, r_mask.cpu().numpy().view(np.uint64))
        assert np.array_equal(g_out, r_out.cpu().numpy())
    mine.close()
    ref.close()


def test_host_policy_differs_from_device_policy_and_caps_an_insert(torch_cuda, reference_gpu):
    """max_modify_size bounds the lines one insert may change under the host policy too, and a device
    key buffer is accepted (copied to the host first)."""
    torch = torch_cuda
    rows = 4000
    t = byte_table(rows, seed=5)
    cache_bytes = 128 * per_set_host()
    mine = CacheTable(cache_bytes, ROW, key_dtype=np.int64, modify_on_gpu=False, max_modify=50)
    ref = reference_gpu.host_cache(cache_bytes, ROW, max_modify=50)
    keys = dg.zipf_keys(3000, rows, 1.05, 9, dg.permutation(rows))
    vals = t[keys]
    v_dev, k_dev = to_dev(torch, vals), to_dev(torch, keys)
    # keys handed over as a device buffer
    mine.table.insert(mine.ctx, keys.size, k_dev.data_ptr(), ROW, ROW, v_dev.data_ptr())
    mine.ctx.wait()
    ref.insert(keys.ctypes.data, keys.size, v_dev.data_ptr(), ROW)
    rt = ref_tags(ref)
    assert (rt != -1).sum() == 50
    assert np.array_equal(mine.tags(), rt)
    mine.close()
    ref.close()


def test_host_policy_modify_ops(torch_cuda, reference_gpu):
    """update, update_accumulate (fp32), invalidate and clear under the host policy; and an insert
    whose rows come from a backing table indexed by key."""
    torch = torch_cuda
    rows, width = 3000, 16
    t = dg.dyadic_table(rows, width, 3, np.float32)
    t_dev = to_dev(torch, t)
    cache_bytes = 64 * per_set_host()
    mine = CacheTable(cache_bytes, ROW, value_dtype="f32", key_dtype=np.int64, modify_on_gpu=False,
                      backing=t_dev.data_ptr(), backing_rows=rows)
    ref = reference_gpu.host_cache(cache_bytes, ROW)
    keys = dg.zipf_keys(1500, rows, 1.1, 7, dg.permutation(rows))
    mine.insert_from_backing(keys)
    ref.insert(keys.ctypes.data, keys.size, t_dev.data_ptr(), ROW, linear=True)
    rt = ref_tags(ref)
    assert np.array_equal(mine.tags(), rt)
    valid = rt != -1
    assert np.array_equal(mine.data()[valid], ref_rows(ref, ROW)[valid])

    uk = np.unique(keys)[:400]
    new = dg.dyadic_table(uk.size, width, 31, np.float32)
    new_dev = to_dev(torch, new)
    mine.update(uk, new.view(np.uint8).reshape(-1, ROW))
    ref.update(uk.ctypes.data, uk.size, new_dev.data_ptr(), ROW)
    assert np.array_equal(mine.data()[valid], ref_rows(ref, ROW)[valid])
    # write-through: the backing table took the new rows as well
    assert np.array_equal(t_dev.cpu().numpy()[uk], new)

    upd = dg.dyadic_table(uk.size, width, 32, np.float32)
    upd_dev = to_dev(torch, upd)
    mine.update_accumulate(uk, upd, "f32")
    ref.update_accumulate(uk.ctypes.data, uk.size, upd_dev.data_ptr(), ROW)
    assert np.array_equal(mine.data()[valid], ref_rows(ref, ROW)[valid])
    assert np.array_equal(t_dev.cpu().numpy()[uk], new + upd)

    gone = np.unique(keys)[100:300]
    mine.erase(gone)
    ref.invalidate(gone.ctypes.data, gone.size)
    assert np.array_equal(mine.tags(), ref_tags(ref))
    # an insert after the erase sees the emptied ways (counters kept, as in the reference)
    more = dg.zipf_keys(900, rows, 1.1, 8, dg.permutation(rows))
    mine.insert_from_backing(more)
    ref.insert(more.ctypes.data, more.size, t_dev.data_ptr(), ROW, linear=True)
    assert np.array_equal(mine.tags(), ref_tags(ref))
    mine.clear()
    ref.clear()
    assert np.array_equal(mine.tags(), ref_tags(ref))
    assert (mine.tags() == -1).all()
    mine.insert_from_backing(more)
    ref.insert(more.ctypes.data, more.size, t_dev.data_ptr(), ROW, linear=True)
    assert np.array_equal(mine.tags(), ref_tags(ref))
    mine.close()
    ref.close()


def test_cache_rows_in_host_memory(torch_cuda, oracle):
    """data_storage_on_host = 1: the rows of the cache live in pinned host memory the GPU maps; tags,
    hit masks and rows read through the cache are those of a cache with rows in HBM."""
    torch = torch_cuda
    rows, width = 3000, 16
    t = dg.dyadic_table(rows, width, 3, np.float32)
    cache_bytes = 64 * per_set()
    hbm = CacheTable(cache_bytes, ROW, value_dtype="f32", key_dtype=np.int64)
    host = CacheTable(cache_bytes, ROW, value_dtype="f32", key_dtype=np.int64, data_storage_on_host=True)
    keys = dg.zipf_keys(1500, rows, 1.1, 7, dg.permutation(rows))
    vals = t[keys].view(np.uint8).reshape(-1, ROW)
    upd = dg.dyadic_table(keys.size, width, 32, np.float32)
    for c in (hbm, host):
        c.insert(keys, vals)
        c.update_accumulate(keys, upd, "f32")       # duplicates of a batch are summed
    assert np.array_equal(hbm.tags(), host.tags())
    valid = hbm.tags() != -1
    assert np.array_equal(hbm.data()[valid], host.data()[valid])
    probe = dg.zipf_keys(1000, rows, 1.1, 8, dg.permutation(rows))
    outs = []
    for c in (hbm, host):
        out, mask = np.zeros((1000, ROW), np.uint8), np.zeros(16, np.uint64)
        c.find(probe, out, mask)
        outs.append((out, mask))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    assert outs[0][1].any()
    hbm.close()
    host.close()
