"""Parity at the benchmark configurations' full sizes.  The tables are generated on the device;
the oracle works on a host mirror of the rows a batch actually touches (rows are re-indexed, which
does not change any result), so full-size batches are checked element for element."""
import ctypes as C

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import ptr, to_dev

pytestmark = pytest.mark.gpu


def touched_mirror(torch, table_dev, keys_np):
    """(compact host table of the touched rows as bytes, keys re-indexed into it)"""
    uniq, inv = np.unique(keys_np, return_inverse=True)
    rows = table_dev[torch.from_numpy(uniq).cuda()].contiguous().cpu().numpy()
    return rows.view(np.uint8).reshape(rows.shape[0], -1), inv.astype(np.int64)


def test_c2_full_table_batch_matches_oracle(torch_cuda, oracle):
    """One table of the headline config: 4M x 128 fp16, 65536 CSR bags of 1..32 keys, Zipf(1.1), mean."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GPUEmbeddingLayer
    rows, dim, bags = 4_000_000, 128, 65_536
    gen = torch.Generator(device="cuda")
    gen.manual_seed(20)
    table = (torch.randn((rows, dim), generator=gen, device="cuda") * 0.02).half()
    _, offs = dg.csr_bags(bags, 1, 32, 1200)
    keys = dg.zipf_keys(int(offs[-1]), rows, 1.1, 6200, dg.permutation(rows))
    layer = GPUEmbeddingLayer(table, rows, dim * 2, "float16")
    ctx = layer.create_execution_context()
    out = torch.zeros((bags, dim), dtype=torch.float16, device="cuda")
    layer.lookup_pooled(ctx, keys.size, to_dev(torch, keys), out, dim * 2, "mean", "float16",
                        csr_offsets=to_dev(torch, offs), num_csr_offsets=offs.size)
    ctx.wait()
    mirror, local = touched_mirror(torch, table, keys)
    want = oracle.lookup_pooled(mirror, "f16", dim, local, "mean", offsets=offs, out_dtype="f16")
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # size-independent property: un-pooled rows of the same keys, summed in fp32 by torch, divided
    rows_out = torch.zeros((keys.size, dim), dtype=torch.float16, device="cuda")
    layer.lookup(ctx, keys.size, to_dev(torch, keys), rows_out, dim * 2)
    ctx.wait()
    seg = torch.repeat_interleave(torch.arange(bags, device="cuda"), torch.from_numpy(np.diff(offs)).cuda())
    acc = torch.zeros((bags, dim), dtype=torch.float32, device="cuda").index_add_(0, seg, rows_out.float())
    mean = (acc / torch.from_numpy(np.diff(offs)).cuda().float()[:, None]).cpu().numpy()
    assert np.max(np.abs(got.astype(np.float32) - mean)) <= 1e-5 + 2 ** -11 * np.abs(mean).max()
    ctx.destroy(); layer.destroy()


def test_c4a_full_batch_dequant_sum_matches_oracle(torch_cuda, oracle):
    """32768 bags x 20 keys over int8 rows with fp32 scale (tight 260-byte rows and padded 272),
    table scaled to 5M rows to keep the test short; the batch has the full size."""
    torch = torch_cuda
    from bench_workloads import _quant_table
    rows, width, bags, hot = 5_000_000, 256, 32_768, 20
    keys = dg.zipf_keys(bags * hot, rows, 1.05, 400)
    d_keys = to_dev(torch, keys)
    for stride in (260, 272):
        t = _quant_table(rows, width, stride, 40)
        out = torch.zeros((bags, width), dtype=torch.float16, device="cuda")
        a = capi.PoolArgs()
        a.table, a.num_rows, a.row_stride = t.data_ptr(), rows, stride
        a.value_dtype, a.row_width, a.default_row_index = capi.DTYPE_QINT8_F32, width, -1
        a.cache, a.key_type, a.keys, a.num_keys = None, capi.KEY_INT64, d_keys.data_ptr(), keys.size
        a.pooling_type, a.sparse_type, a.num_bags, a.fixed_hotness = capi.POOL_SUM, capi.SPARSE_FIXED, bags, hot
        a.output, a.output_stride, a.output_dtype = out.data_ptr(), width * 2, capi.DTYPE_FLOAT16
        capi.check(capi.lib.nve_b200_lookup_pool(C.byref(a), None))
        torch.cuda.synchronize()
        mirror, local = touched_mirror(torch, t, keys)
        want = oracle.lookup_pooled(mirror, "qint8_f32", width, local, "sum", hotness=hot, out_dtype="f16")
        assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16)), stride
        del t


def test_c4b_full_batch_update_matches_oracle(torch_cuda, oracle):
    """1,048,576 (key, grad) pairs, Zipf(1.05), fp32 x 128, SGD lr 0.01 through dedup + fused apply."""
    torch = torch_cuda
    rows, dim, n = 10_000_000, 128, 1_048_576
    gen = torch.Generator(device="cuda")
    gen.manual_seed(50)
    table = torch.empty((rows, dim), dtype=torch.float32, device="cuda").normal_(0, 0.02, generator=gen)
    keys = dg.zipf_keys(n, rows, 1.05, 500)
    grads = torch.empty((n, dim), dtype=torch.float32, device="cuda").normal_(0, 1e-2, generator=gen)
    mirror_before, local = touched_mirror(torch, table, keys)
    d = C.c_void_p()
    capi.check(capi.lib.nve_b200_deduper_create(C.byref(d), capi.KEY_INT64, 1024, n))
    i64 = dict(dtype=torch.int64, device="cuda")
    cap = n + n // 1024 + 2
    uniq, counts, inverse = torch.zeros(n + 1, **i64), torch.zeros(n + 1, **i64), torch.zeros(n + 1, **i64)
    offsets, loc = torch.zeros(cap + 1, **i64), torch.zeros(cap + 1, **i64)
    runs = (C.c_int64 * 2)()
    d_keys = to_dev(torch, keys)
    capi.check(capi.lib.nve_b200_deduper_dedup(d, ptr(d_keys), n, ptr(uniq), ptr(counts), ptr(loc), runs,
                                               ptr(inverse), ptr(offsets), None, 24))
    u = int(runs[0])
    o = oracle.dedup(keys, max_run=1024)
    assert u == o["num_unique"] and int(runs[1]) == o["num_chunks"]
    assert np.array_equal(uniq[:u].cpu().numpy(), o["unique"])
    assert np.array_equal(counts[:u].cpu().numpy(), o["counts"])
    assert np.array_equal(inverse[:n].cpu().numpy(), o["inverse"])
    capi.check(capi.lib.nve_b200_dedup_grads(d, ptr(grads), dim * 4, dim * 4, n, ptr(uniq), ptr(inverse),
                                             ptr(offsets), ptr(loc), ptr(table), dim * 4, 1, rows, -0.01, None))
    torch.cuda.synchronize()
    got = table[torch.from_numpy(o["unique"]).cuda()].cpu().numpy()
    upd = (np.float32(-0.01) * oracle.dedup_grads(grads.cpu().numpy(), o)).astype(np.float32)
    want = mirror_before.view(np.float32).reshape(u, dim).copy()
    oracle.update_accumulate(want, np.arange(u, dtype=np.int64), upd)
    assert np.array_equal(got, want)
    exact = mirror_before.view(np.float32).reshape(u, dim).astype(np.float64)
    np.add.at(exact, local, -0.01 * grads.cpu().numpy().astype(np.float64))
    assert np.max(np.abs(got - exact) / np.maximum(np.abs(exact), 1e-2)) <= 1e-6 * 20
    capi.check(capi.lib.nve_b200_deduper_destroy(d))


def test_dedup_properties_at_full_size(torch_cuda):
    """1 048 576 keys (the C4b batch): properties that hold whatever the keys are — unique keys
    strictly ascending, counts sum to n, the inverse buffer is a permutation whose keys are grouped
    exactly as (unique, counts) say, positions ascend inside a group, chunks respect max_run and
    tile the groups."""
    torch = torch_cuda
    n, rows, max_run = 1_048_576, 10_000_000, 1024
    keys = to_dev(torch, dg.zipf_keys(n, rows, 1.05, 500))
    d = C.c_void_p()
    capi.check(capi.lib.nve_b200_deduper_create(C.byref(d), capi.KEY_INT64, max_run, n))
    i64 = dict(dtype=torch.int64, device="cuda")
    cap = n + n // max_run + 2
    uniq, counts, inverse = torch.empty(n + 1, **i64), torch.empty(n + 1, **i64), torch.empty(n + 1, **i64)
    offsets, loc = torch.empty(cap + 1, **i64), torch.empty(cap + 1, **i64)
    runs = (C.c_int64 * 2)()
    capi.check(capi.lib.nve_b200_deduper_dedup(d, keys.data_ptr(), n, uniq.data_ptr(), counts.data_ptr(),
                                               loc.data_ptr(), runs, inverse.data_ptr(), offsets.data_ptr(),
                                               None, 24))
    u, c = runs[0], runs[1]
    uq, ct, inv, off, lm = uniq[:u], counts[:u], inverse[:n], offsets[:c + 1], loc[:c]
    assert bool((uq[1:] > uq[:-1]).all())
    assert int(ct.sum()) == n and int(ct.min()) >= 1
    assert bool((torch.sort(inv).values == torch.arange(n, device="cuda")).all())
    assert bool((keys[inv] == torch.repeat_interleave(uq, ct)).all())
    starts = torch.cumsum(ct, 0) - ct
    same_group = torch.ones(n, dtype=torch.bool, device="cuda")
    same_group[starts] = False
    assert bool((inv[1:][same_group[1:]] > inv[:-1][same_group[1:]]).all())     # stable: ascending positions
    lens = off[1:] - off[:-1]
    assert int(off[0]) == 0 and int(off[-1]) == n and int(lens.max()) <= max_run and int(lens.min()) >= 1
    per_group = torch.bincount(lm, minlength=u)
    assert bool((per_group == (ct + max_run - 1) // max_run).all())
    assert bool((off[:-1][torch.cat([torch.ones(1, dtype=torch.bool, device="cuda"), lm[1:] != lm[:-1]])] == starts).all())
    capi.check(capi.lib.nve_b200_deduper_destroy(d))


def test_pooled_sum_is_linear_in_the_table_at_full_size(torch_cuda):
    """C2's shape with exactly summable (dyadic) fp32 rows: pooled(T1 + T2) == pooled(T1) + pooled(T2)
    bit for bit, and a weighted sum with all weights 2 is twice the plain sum."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GPUEmbeddingLayer
    rows, dim, bags = 4_000_000, 128, 65_536
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)

    def dyadic():
        a = torch.randint(-8, 9, (rows, dim), generator=gen, device="cuda", dtype=torch.int32).float()
        b = torch.randint(3, 10, (rows, dim), generator=gen, device="cuda", dtype=torch.int32).float()
        return a / torch.exp2(b)
    t1, t2 = dyadic(), dyadic()
    _, offs = dg.csr_bags(bags, 1, 32, 1300)
    keys = to_dev(torch, dg.zipf_keys(int(offs[-1]), rows, 1.1, 6300, dg.permutation(rows)))
    d_offs = to_dev(torch, offs)

    def pooled(table, weights=None):
        layer = GPUEmbeddingLayer(table, rows, dim * 4, "float32")
        ctx = layer.create_execution_context()
        out = torch.zeros((bags, dim), dtype=torch.float32, device="cuda")
        layer.lookup_pooled(ctx, keys.numel(), keys, out, dim * 4, "sum" if weights is None else "weighted_sum",
                            "float32", csr_offsets=d_offs, num_csr_offsets=offs.size, weights=weights,
                            weight_type="float32")
        ctx.wait()
        ctx.destroy(); layer.destroy()
        return out
    p1, p2 = pooled(t1), pooled(t2)
    t1.add_(t2)
    p12 = pooled(t1)
    assert bool(torch.equal(p12, p1 + p2))
    w = torch.full((keys.numel(),), 2.0, device="cuda")
    assert bool(torch.equal(pooled(t1, w), 2 * p12))


def test_cache_insert_is_idempotent_at_c3_batch_size(torch_cuda):
    """Inserting the same 262 144-key batch twice leaves every tag where it was (all keys of the
    second insert are resident or lose to resident keys exactly as before)."""
    torch = torch_cuda
    from nve_helpers import CacheTable
    rows, row_bytes, batch = 8_000_000, 256, 262_144
    table = torch.randint(0, 256, (rows, row_bytes), dtype=torch.uint8, device="cuda")
    cache = CacheTable(int(rows * 0.1) * row_bytes, row_bytes, backing=table, backing_rows=rows,
                       max_modify=batch)
    keys = dg.zipf_keys(batch, rows, 1.2, 300)
    cache.insert_from_backing(keys)
    tags1 = cache.tags().copy()
    cache.insert_from_backing(keys)
    tags2 = cache.tags()
    assert np.array_equal(tags1, tags2)
    resident = int((tags1 != -1).sum())            # a tag is key / num_sets: count the occupied ways
    assert resident > 10_000
    out = np.zeros((1000, row_bytes), np.uint8)
    probe = keys[:1000]
    cache.find(probe, out, None)
    hit = ~np.all(out == 0, axis=1)
    assert hit.any() and np.array_equal(out[hit], table[torch.from_numpy(probe[hit]).cuda()].cpu().numpy())
    cache.close()


def test_c3_full_batch_cached_gather_matches_oracle_cache(torch_cuda, oracle):
    """The cached-layer configuration at its own batch size and cache fraction: a table of fp16 rows
    in pinned host memory (scaled to 4 M rows), a cache of 10 % of its rows warmed by 20 inserts of
    262 144 Zipf(1.2) keys, then one lookup of 262 144 Zipf(1.2) keys and one of uniform keys.  Rows
    byte-exact; resident tags of every (set, way) and the miss counts equal to the oracle cache that
    saw the same inserts."""
    torch = torch_cuda
    from nve_helpers import CacheTable
    from oracle.pyoracle import OracleCache
    rows, dim, batch = 4_000_000, 128, 262_144
    row_bytes = dim * 2
    tb = np.random.default_rng(30).integers(0, 256, (rows, row_bytes), dtype=np.uint8)   # rows are copied as bytes
    backing = torch.from_numpy(tb).pin_memory()
    cache_bytes = int(rows * 0.10) * row_bytes
    gpu = CacheTable(cache_bytes, row_bytes, value_dtype="f16", backing=backing, backing_rows=rows, max_modify=batch)
    ref = OracleCache(oracle, cache_bytes, row_bytes)
    assert gpu.num_sets == ref.num_sets
    for b in range(20):
        keys = dg.zipf_keys(batch, rows, 1.2, 300 + b)
        gpu.insert_from_backing(keys)
        ref.insert(keys, table=tb, max_modify=batch)
    assert np.array_equal(gpu.tags(), ref.tags())
    for name, keys in (("zipf", dg.zipf_keys(batch, rows, 1.2, 320)), ("uniform", dg.uniform_keys(batch, rows, 321))):
        out = np.zeros((batch, row_bytes), np.uint8)
        misses = gpu.find(keys, out)
        assert np.array_equal(out, tb[keys]), name
        ref.reset_misses()
        ref.lookup(keys, None)
        assert misses == ref.misses, (name, misses, ref.misses)
        hit_rate = 1.0 - misses / batch
        assert (hit_rate > 0.8) if name == "zipf" else (hit_rate < 0.3), (name, hit_rate)
    gpu.close()


def test_c1_host_layer_configuration_on_the_gpu(torch_cuda, oracle):
    """The reference's CPU-runnable configuration with its own inputs: one table of 1 000 000 x 64
    fp32 uniform[-0.05, 0.05] (seed 1), 8192 bags at a fixed pooling factor of 16, Zipf(1.05) keys over
    a permuted row order, fp32 sums.  The dense layer on the GPU must give the oracle's bits (the
    oracle is pinned to the reference's HostEmbeddingLayer on exactly this shape)."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GPUEmbeddingLayer
    rows, dim, bags, hot = 1_000_000, 64, 8192, 16
    table_np = np.random.default_rng(1).uniform(-0.05, 0.05, (rows, dim)).astype(np.float32)
    keys = dg.zipf_keys(bags * hot, rows, 1.05, 1000, dg.permutation(rows))
    table = torch.from_numpy(table_np).cuda()
    layer = GPUEmbeddingLayer(table, rows, dim * 4, "float32")
    ctx = layer.create_execution_context()
    out = torch.zeros((bags, dim), dtype=torch.float32, device="cuda")
    layer.lookup_pooled(ctx, keys.size, to_dev(torch, keys), out, dim * 4, "sum", "float32", fixed_hotness=hot)
    ctx.wait()
    want = oracle.lookup_pooled(table_np.view(np.uint8).reshape(rows, -1), "f32", dim, keys, "sum", hotness=hot,
                                out_dtype="f32")
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # host buffers in, host buffer out: the call a CPU user of the reference layer makes
    out_h = np.zeros((bags, dim), np.float32)
    layer.lookup_pooled(ctx, keys.size, keys, out_h, dim * 4, "sum", "float32", fixed_hotness=hot)
    ctx.wait()
    assert np.array_equal(out_h.view(np.uint32), want.view(np.uint32))
    ctx.destroy(); layer.destroy()
