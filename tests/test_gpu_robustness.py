"""GPU checks of paths that inputs outside the happy case reach: keys that are no rows of the
backing table on the automatic-insert path and in nve_b200_gpu_table_insert_from_backing, duplicate
keys in update_accumulate of the cached table, lookups and automatic inserts on distinct
non-blocking streams, and the status word of the gradient reduction."""
import ctypes as C

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import CacheTable, device_read, to_dev
from oracle.pyoracle import OracleCache

pytestmark = pytest.mark.gpu

ROW = 64


def per_set(row=ROW, key_bytes=8):
    return 8 * key_bytes + 8 * row + 32


def resident_tags(gt, ctx, key_bytes=8):
    view = capi.CacheData()
    capi.check(capi.lib.nve_b200_gpu_table_get_cache_data(gt.handle, ctx.handle, C.byref(view)))
    raw = device_read(view.tags_ptr, view.num_sets * 8 * key_bytes)
    tags = raw.view(np.int64).reshape(view.num_sets, 8)
    sets = np.arange(view.num_sets, dtype=np.int64)[:, None]
    keys = tags * view.num_sets + sets
    return keys[tags != -1]


def test_auto_insert_ignores_keys_outside_the_table(torch_cuda):
    """Keys -1 and num_rows + 5 are legal in a lookup with a default row.  The automatic insert
    must neither read the backing table at those indices nor make them resident: afterwards they
    still read the default row, and every resident key is a row of the table."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GpuTable, LinearUVMEmbeddingLayer
    rows, dim, default_row = 20000, 64, 11
    table = dg.normal_table(rows, dim, 0.02, 1, np.float16)
    backing = torch.from_numpy(table).pin_memory()
    cache_bytes = (4000 // 8) * per_set(dim * 2)
    gt = GpuTable(cache_bytes, dim * 2, "float16", uvm_table=backing, uvm_num_rows=rows)
    layer = LinearUVMEmbeddingLayer(gt, default_row_index=default_row, insert_heuristic="default",
                                    min_insert_size_gpu=2000)
    # lookups and inserts on two distinct non-blocking streams
    s_lookup, s_modify = torch.cuda.Stream(), torch.cuda.Stream()
    ctx = layer.create_execution_context(s_lookup.cuda_stream, s_modify.cuda_stream)
    perm = dg.permutation(rows)
    rates = []
    for step in range(16):
        keys = dg.zipf_keys(5000, rows, 1.2, 40 + step, perm)
        keys[::7] = -1
        keys[3::11] = rows + 5
        keys[5::13] = -(1 << 40)
        keys[1::17] = rows + (1 << 33) + 3      # same low bits as row 3
        d_keys = to_dev(torch, keys)
        out = torch.zeros((5000, dim), dtype=torch.float16, device="cuda")
        with torch.cuda.stream(s_lookup):
            rates.append(layer.lookup(ctx, keys.size, d_keys, out, dim * 2, want_hitrate=True))
        ctx.wait()
        want = table[np.where((keys >= 0) & (keys < rows), keys, default_row)]
        assert np.array_equal(out.cpu().numpy(), want), step
    assert max(rates[3:]) > 0.3, rates          # inserts did happen
    torch.cuda.synchronize()
    resident = resident_tags(gt, ctx)
    assert resident.size > 0
    assert resident.min() >= 0 and resident.max() < rows
    assert np.unique(resident).size == resident.size
    ctx.destroy(); layer.destroy(); gt.destroy()


def test_insert_from_backing_drops_keys_outside_the_table(torch_cuda, oracle):
    torch = torch_cuda
    rows = 3000
    t = np.random.default_rng(5).integers(0, 256, (rows, ROW), dtype=np.uint8)
    backing = torch.from_numpy(t).cuda()
    gpu = CacheTable(64 * per_set(), ROW, backing=backing, backing_rows=rows)
    ref = OracleCache(oracle, 64 * per_set(), ROW)
    keys = dg.zipf_keys(1500, rows, 1.05, 9, dg.permutation(rows))
    dirty = keys.copy()
    dirty = np.concatenate([dirty, np.array([-1, -5, rows, rows + 7, rows + (1 << 32) + keys[0]], np.int64)])
    gpu.insert_from_backing(dirty)
    # the reference sees only the rows of the table; priorities are counts over the batch size
    ref.insert(keys, table=t)
    gt, rt = gpu.tags(), ref.tags()
    assert np.array_equal(gt, rt)
    valid = rt != -1
    assert np.array_equal(gpu.data()[valid], ref.data()[valid])
    gpu.close()


@pytest.mark.parametrize("dtype,npdt", [("f32", np.float32), ("f16", np.float16)])
def test_accumulate_sums_duplicate_keys(torch_cuda, dtype, npdt):
    """A batch may name a key several times (direct C-ABI callers do not coalesce): every update
    is added, in the cache line and in the backing table.  Dyadic values keep the sums exact."""
    torch = torch_cuda
    rows, width = 400, 32
    row_bytes = width * np.dtype(npdt).itemsize
    tf = (np.round(np.random.default_rng(2).normal(size=(rows, width)) * 8) / 8).astype(npdt)
    backing = torch.from_numpy(tf.view(np.uint8).reshape(rows, row_bytes).copy()).cuda()
    gpu = CacheTable(16 * per_set(row_bytes), row_bytes, value_dtype=dtype, backing=backing, backing_rows=rows)
    gpu.insert_from_backing(np.arange(0, 120, dtype=np.int64))
    keys = np.random.default_rng(3).integers(0, 200, 600).astype(np.int64)      # many repeats
    upd = (np.round(np.random.default_rng(4).normal(size=(600, width)) * 4) / 4).astype(npdt)
    gpu.update_accumulate(keys, upd, dtype)
    want = tf.astype(np.float64)
    np.add.at(want, keys, upd.astype(np.float64))
    got_backing = backing.cpu().numpy().view(npdt).reshape(rows, width)
    assert np.array_equal(got_backing.astype(np.float64), want)
    out = np.zeros((rows, row_bytes), np.uint8)
    gpu.find(np.arange(rows, dtype=np.int64), out)
    assert np.array_equal(out.view(npdt).reshape(rows, width).astype(np.float64), want)
    gpu.close()


def test_gradient_reduction_status_word(torch_cuda):
    """nve_b200_dedup_grads_status reads and clears the overflow flag of the partial-sum scratch;
    a regular reduction leaves it clear."""
    torch = torch_cuda
    n, gw = 6000, 64
    keys = dg.zipf_keys(n, 50, 1.05, 6, dg.permutation(50))
    grads = np.random.default_rng(7).normal(0, 1e-2, (n, gw)).astype(np.float32)
    d = C.c_void_p()
    capi.check(capi.lib.nve_b200_deduper_create(C.byref(d), capi.KEY_INT64, 64, n))
    i64 = dict(dtype=torch.int64, device="cuda")
    uniq, counts, inverse = torch.empty(n + 1, **i64), torch.empty(n + 1, **i64), torch.empty(n + 1, **i64)
    cap = n + n // 64 + 8
    offs, loc = torch.empty(cap, **i64), torch.empty(cap, **i64)
    runs = (C.c_int64 * 2)()
    gk, gg = to_dev(torch, keys), to_dev(torch, grads)
    capi.check(capi.lib.nve_b200_deduper_dedup(d, gk.data_ptr(), n, uniq.data_ptr(), counts.data_ptr(),
                                               loc.data_ptr(), runs, inverse.data_ptr(), offs.data_ptr(), None, 0))
    sums = torch.zeros((runs[0], gw), device="cuda")
    capi.check(capi.lib.nve_b200_dedup_grads(d, gg.data_ptr(), gw * 4, gw * 4, n, uniq.data_ptr(),
                                             inverse.data_ptr(), offs.data_ptr(), loc.data_ptr(), sums.data_ptr(),
                                             gw * 4, 0, 0, 1.0, None))
    flag = C.c_int32(-1)
    capi.check(capi.lib.nve_b200_dedup_grads_status(C.byref(flag)))
    assert flag.value == 0
    capi.check(capi.lib.nve_b200_deduper_destroy(d))


def test_host_resident_csr_offsets_are_validated_before_any_launch(torch_cuda):
    """Offsets in host memory that do not start at 0, decrease, or do not end at the number of keys are
    refused with INVALID_ARGUMENT (what the reference's CPU path enforces); the same offsets in device
    memory are the caller's responsibility, as in the reference's GPU path."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GPUEmbeddingLayer
    rows, dim = 1000, 16
    table = to_dev(torch, dg.normal_table(rows, dim, 0.02, 1, np.float16))
    layer = GPUEmbeddingLayer(table, rows, dim * 2, "float16")
    ctx = layer.create_execution_context()
    keys = np.arange(40, dtype=np.int64)
    out = np.zeros((4, dim), np.float16)
    good = np.array([0, 10, 20, 30, 40], np.int64)
    layer.lookup_pooled(ctx, 40, keys, out, dim * 2, "sum", "float16", csr_offsets=good, num_csr_offsets=5)
    ctx.wait()
    for bad, what in ((np.array([1, 10, 20, 30, 40], np.int64), "start at 0"),
                      (np.array([0, 20, 10, 30, 40], np.int64), "decrease"),
                      (np.array([0, 10, 20, 30, 41], np.int64), "last CSR offset")):
        with pytest.raises(capi.NveError) as e:
            layer.lookup_pooled(ctx, 40, keys, out, dim * 2, "sum", "float16", csr_offsets=bad, num_csr_offsets=5)
        assert e.value.status == capi.NVE_ERROR_INVALID_ARGUMENT and what in e.value.message
    ctx.wait()
    ctx.destroy(); layer.destroy()


CHECKED = r'''
import os, sys
import numpy as np, torch
sys.path.insert(0, os.environ["NVE_ROOT"])
from nv_embedding_cache_b200 import capi, datagen as dg
from nv_embedding_cache_b200.layers import GPUEmbeddingLayer
assert capi._LIB_PATH.name == "libnve_b200_checked.so"
rows, dim = 5000, 64
table_np = dg.normal_table(rows, dim, 0.02, 1, np.float16)
# room behind the table, so that an index a few rows past the end stays inside the allocation even
# if a check were missing
store = torch.zeros((rows + 64, dim), dtype=torch.float16, device="cuda")
store[:rows] = torch.from_numpy(table_np).cuda()
layer = GPUEmbeddingLayer(store, rows, dim * 2, "float16")          # no default row
ctx = layer.create_execution_context()
keys = dg.uniform_keys(64 * 8, rows, 3)
d_keys = torch.from_numpy(keys).cuda()
out = torch.zeros((64, dim), dtype=torch.float16, device="cuda")
layer.lookup_pooled(ctx, keys.size, d_keys, out, dim * 2, "sum", "float16", fixed_hotness=8)
ctx.wait()                                                            # clean inputs: no report
want = table_np[keys].astype(np.float32).reshape(64, 8, dim)
acc = np.zeros((64, dim), np.float32)
for j in range(8):
    acc = acc + want[:, j]
assert np.array_equal(out.cpu().numpy(), acc.astype(np.float16))
codes = []
# (a) keys that are no rows of the table: read as row 0, reported
bad = keys.copy(); bad[5] = rows + 3; bad[77] = rows + 40
layer.lookup_pooled(ctx, bad.size, torch.from_numpy(bad).cuda(), out, dim * 2, "sum", "float16", fixed_hotness=8)
try:
    ctx.wait(); codes.append("no report")
except capi.NveError as e:
    codes.append("keys" if "no rows of a table" in e.message else e.message)
# (b) device-resident offsets that run past the keys: that bag pools to zeros, reported
offs = torch.tensor([0, 8, 16, 24, keys.size + 100], dtype=torch.int64, device="cuda")
out4 = torch.ones((4, dim), dtype=torch.float16, device="cuda")
layer.lookup_pooled(ctx, keys.size, d_keys, out4, dim * 2, "sum", "float16", csr_offsets=offs, num_csr_offsets=5)
try:
    ctx.wait(); codes.append("no report")
except capi.NveError as e:
    codes.append("offsets" if "CSR offsets" in e.message else e.message)
assert not out4[3].any().item() and out4[0].any().item()
# (c) the report is one-shot: a clean lookup afterwards waits without error
layer.lookup_pooled(ctx, keys.size, d_keys, out, dim * 2, "sum", "float16", fixed_hotness=8)
ctx.wait()
# (d) host-resident keys of a table without a default row are refused before the launch
try:
    layer.lookup_pooled(ctx, bad.size, bad, out, dim * 2, "sum", "float16", fixed_hotness=8); codes.append("launched")
except capi.NveError as e:
    codes.append("host keys" if e.status == capi.NVE_ERROR_INVALID_ARGUMENT else e.message)
print(codes)
sys.exit(0 if codes == ["keys", "offsets", "host keys"] else 3)
'''


def test_checked_build_reports_instead_of_reading_out_of_bounds(torch_cuda, tmp_path):
    """libnve_b200_checked.so (the -DNVE_B200_BOUNDS_CHECK build, loaded through NVE_B200_LIBRARY in a
    process of its own): keys outside a table without a default row and offsets outside the keys are
    left out and reported at nve_context_wait."""
    import os, subprocess, sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    lib = root / "nv_embedding_cache_b200" / "libnve_b200_checked.so"
    assert lib.exists(), "build it with python -m nv_embedding_cache_b200.build --bounds-check"
    script = tmp_path / "checked.py"
    script.write_text(CHECKED)
    env = dict(os.environ, NVE_ROOT=str(root), NVE_B200_LIBRARY=str(lib))
    res = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
