"""GPU checks of the cached layer over a linear backing table (pinned host memory, a managed block
kept in host memory, and device memory) and of the pynve-named Python edge, against the oracle.  Outputs never depend on what is
cached; hit rates must equal the oracle cache's."""
import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import to_dev
from oracle.pyoracle import OracleCache

pytestmark = pytest.mark.gpu


def make_layer(torch, table_np, cache_rows, where, dtype="float16", default_row=-1):
    from nv_embedding_cache_b200.layers import GpuTable, LinearUVMEmbeddingLayer
    rows, row_bytes = table_np.shape[0], table_np.strides[0]
    if where == "managed":
        from nv_embedding_cache_b200.memblock import ManagedMemBlock
        backing = ManagedMemBlock(table_np.nbytes, (0,))
        backing.copy_from(table_np)
        assert backing.get_type() == "Managed" and backing.get_size_in_bytes() == table_np.nbytes
        assert backing.get_handle() == backing.data_ptr()
    elif where == "host":
        backing = torch.from_numpy(table_np).pin_memory()
    else:
        backing = torch.from_numpy(table_np).cuda()
    cache_bytes = (cache_rows // 8) * (64 + 8 * row_bytes + 32)
    gt = GpuTable(cache_bytes, row_bytes, dtype, uvm_table=backing, uvm_num_rows=rows)
    layer = LinearUVMEmbeddingLayer(gt, default_row_index=default_row)
    return layer, gt, backing, cache_bytes


@pytest.mark.parametrize("where", ["host", "device", "managed"])
def test_unpooled_lookup_is_byte_exact_and_hitrate_matches(torch_cuda, oracle, where):
    torch = torch_cuda
    rows, dim = 20000, 128
    table = dg.normal_table(rows, dim, 0.02, 1, np.float16)
    layer, gt, backing, cache_bytes = make_layer(torch, table, 2000, where)
    ctx = layer.create_execution_context()
    ref = OracleCache(oracle, cache_bytes, dim * 2)
    tb = table.view(np.uint8).reshape(rows, -1)
    perm = dg.permutation(rows)
    for step in range(4):
        warm = dg.zipf_keys(3000, rows, 1.2, 10 + step, perm)
        layer.insert(ctx, warm.size, warm, dim * 2, dim * 2, tb[warm])   # host buffers
        ctx.wait()
        ref.insert(warm, values=tb[warm])
        keys = dg.zipf_keys(5000, rows, 1.2, 20 + step, perm)
        out = np.zeros((5000, dim), np.float16)
        hr = layer.lookup(ctx, keys.size, keys, out, dim * 2, want_hitrate=True)
        ctx.wait()
        assert np.array_equal(out, table[keys])
        ref.reset_misses()
        ref.lookup(keys, None)
        assert abs(hr - (1.0 - ref.misses / keys.size)) < 1e-6
        assert 0.2 < hr < 1.0
    # uniform keys: a miss-heavy batch, still exact
    keys = dg.uniform_keys(5000, rows, 99)
    d_keys = to_dev(torch, keys)
    d_out = torch.zeros((5000, dim), dtype=torch.float16, device="cuda")
    hr = layer.lookup(ctx, keys.size, d_keys, d_out, dim * 2, want_hitrate=True)
    ctx.wait()
    assert np.array_equal(d_out.cpu().numpy(), table[keys]) and hr < 0.5
    ctx.destroy(); layer.destroy(); gt.destroy()


@pytest.mark.parametrize("pooling,ref_pool", [("sum", "sum"), ("mean", "mean"), ("weighted_sum", "wsum")])
def test_pooled_lookup_through_the_cache(torch_cuda, oracle, pooling, ref_pool):
    torch = torch_cuda
    rows, dim = 10000, 64
    table = dg.normal_table(rows, dim, 0.02, 2, np.float32)
    layer, gt, backing, _ = make_layer(torch, table, 1024, "host", dtype="float32", default_row=7)
    ctx = layer.create_execution_context()
    tb = table.view(np.uint8).reshape(rows, -1)
    warm = dg.zipf_keys(4000, rows, 1.1, 3, dg.permutation(rows))
    layer.insert(ctx, warm.size, warm, dim * 4, dim * 4, tb[warm])
    _, offs = dg.csr_bags(500, 0, 40, 4)
    keys = dg.zipf_keys(int(offs[-1]), rows, 1.1, 5, dg.permutation(rows))
    keys[::97] = -3                                # redirected to the default row
    w = np.random.default_rng(6).uniform(-1, 1, keys.size).astype(np.float32)
    out = np.zeros((500, dim), np.float32)
    hr = layer.lookup_pooled(ctx, keys.size, keys, out, dim * 4, pooling, "float32", csr_offsets=offs,
                             num_csr_offsets=offs.size, weights=w if pooling.startswith("w") else None,
                             weight_type=capi.DTYPE_FLOAT32, want_hitrate=True)
    ctx.wait()
    want = oracle.lookup_pooled(tb, "f32", dim, keys, ref_pool, offsets=offs,
                                weights=w if pooling.startswith("w") else None, default_row=7)
    assert np.array_equal(out, want)
    assert 0.0 < hr < 1.0
    ctx.destroy(); layer.destroy(); gt.destroy()


def test_layer_rejects_hitmask_and_bad_default_row(torch_cuda):
    torch = torch_cuda
    table = dg.normal_table(100, 16, 0.02, 1, np.float16)
    layer, gt, backing, _ = make_layer(torch, table, 64, "device")
    ctx = layer.create_execution_context()
    keys = np.arange(10, dtype=np.int64)
    out = np.zeros((10, 16), np.float16)
    mask = np.zeros(1, np.uint64)
    with pytest.raises(capi.NveError) as e:
        layer.lookup(ctx, 10, keys, out, 32, hitmask=mask)
    assert e.value.status == capi.NVE_ERROR_INVALID_ARGUMENT and "Hitmask" in e.value.message
    from nv_embedding_cache_b200.layers import LinearUVMEmbeddingLayer
    with pytest.raises(capi.NveError):
        LinearUVMEmbeddingLayer(gt, default_row_index=100)
    ctx.destroy(); layer.destroy(); gt.destroy()


@pytest.mark.parametrize("heuristic,expect_hits", [("default", True), (0.5, True), ("never", False)])
def test_automatic_cache_population(torch_cuda, heuristic, expect_hits):
    """No explicit insert: with the default heuristic the layer promotes the keys of looked-up
    batches on its own (hit rate climbs from 0), with the never-insert heuristic the cache stays
    empty.  Rows are exact either way, whatever is resident at the moment."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GpuTable, LinearUVMEmbeddingLayer
    rows, dim = 20000, 128
    table = dg.normal_table(rows, dim, 0.02, 1, np.float16)
    backing = torch.from_numpy(table).pin_memory()
    cache_bytes = (4000 // 8) * (64 + 8 * dim * 2 + 32)
    gt = GpuTable(cache_bytes, dim * 2, "float16", uvm_table=backing, uvm_num_rows=rows)
    layer = LinearUVMEmbeddingLayer(gt, insert_heuristic=heuristic, min_insert_size_gpu=2000)
    ctx = layer.create_execution_context()
    perm = dg.permutation(rows)
    rates = []
    for step in range(14):
        keys = dg.zipf_keys(5000, rows, 1.2, 40 + step, perm)
        d_keys = to_dev(torch, keys)
        out = torch.zeros((5000, dim), dtype=torch.float16, device="cuda")
        rates.append(layer.lookup(ctx, keys.size, d_keys, out, dim * 2, want_hitrate=True))
        ctx.wait()
        assert np.array_equal(out.cpu().numpy(), table[keys])
    assert rates[0] == 0.0
    if expect_hits:
        assert max(rates[3:]) > 0.3, rates
    else:
        assert max(rates) == 0.0, rates
    ctx.destroy(); layer.destroy(); gt.destroy()


def test_pynve_named_edge(torch_cuda, oracle):
    """GPUEmbedding / LinearUVMEmbedding with raw addresses and stream handles, as pynve passes them."""
    torch = torch_cuda
    from nv_embedding_cache_b200 import pynve
    rows, dim = 5000, 32
    table = dg.dyadic_table(rows, dim, 3, np.float32)
    t_dev = to_dev(torch, table)
    emb = pynve.GPUEmbedding(dim, rows, pynve.DataType_t.Float32, t_dev, 0, pynve.EmbedLayerConfig())
    stream = torch.cuda.current_stream().cuda_stream
    _, offs = dg.csr_bags(64, 1, 9, 1)
    keys = dg.uniform_keys(int(offs[-1]), rows, 2)
    d_keys, d_offs = to_dev(torch, keys), to_dev(torch, offs)
    out = torch.zeros((64, dim), device="cuda")
    emb.lookup_with_pooling(keys.size, d_keys.data_ptr(), out.data_ptr(), pynve.PoolingType_t.Sum,
                            offs.size, d_offs.data_ptr(), pynve.DataType_t.Float32, 0, stream)
    torch.cuda.synchronize()
    want = oracle.lookup_pooled(table.view(np.uint8).reshape(rows, -1), "f32", dim, keys, "sum", offsets=offs)
    assert np.array_equal(out.cpu().numpy(), want)
    rows_out = torch.zeros((keys.size, dim), device="cuda")
    emb.lookup(keys.size, d_keys.data_ptr(), rows_out.data_ptr(), stream)
    torch.cuda.synchronize()
    assert np.array_equal(rows_out.cpu().numpy(), table[keys])
    # backward of the un-pooled lookup: unique keys + summed gradient rows, then SGD through accumulate
    grads = dg.dyadic_table(keys.size, dim, 4, np.float32)
    d_grads = to_dev(torch, grads)
    uniq = torch.zeros(keys.size, dtype=torch.int64, device="cuda")
    ugrad = torch.zeros((keys.size, dim), device="cuda")
    nu = emb.concat_backprop(keys.size, d_keys.data_ptr(), d_grads.data_ptr(), uniq.data_ptr(),
                             ugrad.data_ptr(), stream)
    u_np = np.unique(keys)
    assert nu == u_np.size and np.array_equal(uniq[:nu].cpu().numpy(), u_np)
    want_g = np.zeros((nu, dim), np.float64)
    np.add.at(want_g, np.searchsorted(u_np, keys), grads.astype(np.float64))
    assert np.array_equal(ugrad[:nu].cpu().numpy().astype(np.float64), want_g)
    upd = (-0.5 * ugrad[:nu]).contiguous()
    emb.accumulate(nu, uniq.data_ptr(), upd.data_ptr(), stream)
    torch.cuda.synchronize()
    want_t = table.astype(np.float64)
    want_t[u_np] += -0.5 * want_g
    assert np.array_equal(t_dev.cpu().numpy().astype(np.float64), want_t)
    emb.close()


@pytest.mark.parametrize("host_rows", [False, True])
def test_cached_layer_over_the_host_side_policy(torch_cuda, host_rows):
    """A cached layer whose table decides replacements on the host (modify_on_gpu = 0), with the
    cached rows in HBM or in pinned host memory: lookups are exact whatever is cached, explicit
    inserts, updates and the automatic inserts (whose keys are collected on the device) all go through
    the host mirror, and the cache does fill."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GpuTable, LinearUVMEmbeddingLayer
    rows, dim = 20000, 64
    table = dg.normal_table(rows, dim, 0.02, 1, np.float16)
    backing = torch.from_numpy(table).cuda()
    gt = GpuTable(2000 // 8 * (64 + 8 * dim * 2), dim * 2, "float16", uvm_table=backing, uvm_num_rows=rows,
                  modify_on_gpu=False, data_storage_on_host=host_rows)
    layer = LinearUVMEmbeddingLayer(gt)
    ctx = layer.create_execution_context()
    perm = dg.permutation(rows)
    tb = table.view(np.uint8).reshape(rows, -1)
    rates = []
    for step in range(6):
        if step == 1:
            warm = dg.zipf_keys(3000, rows, 1.2, 10, perm)
            layer.insert(ctx, warm.size, warm, dim * 2, dim * 2, tb[warm])
            ctx.wait()
        keys = dg.zipf_keys(70000, rows, 1.2, 20 + step, perm)     # enough keys to trigger automatic inserts
        out = np.zeros((keys.size, dim), np.float16)
        rates.append(layer.lookup(ctx, keys.size, keys, out, dim * 2, want_hitrate=True))
        ctx.wait()
        assert np.array_equal(out, table[keys])
    assert rates[0] == 0.0 and rates[-1] > 0.3, rates
    # an update reaches the cached copy and the backing table
    uk = np.unique(dg.zipf_keys(500, rows, 1.2, 20, perm))
    new = dg.normal_table(uk.size, dim, 0.02, 2, np.float16)
    layer.update(ctx, uk.size, uk, dim * 2, dim * 2, new, -1)
    ctx.wait()
    out = np.zeros((uk.size, dim), np.float16)
    layer.lookup(ctx, uk.size, uk, out, dim * 2)
    ctx.wait()
    assert np.array_equal(out, new)
    assert np.array_equal(backing.cpu().numpy()[uk], new)
