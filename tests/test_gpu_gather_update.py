"""GPU parity of the un-pooled gather family and the row update kernels (dense table layer)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from golden.cases import build_cases
from nv_embedding_cache_b200 import datagen as dg
from nve_helpers import DT, GpuLayer, ptr, to_dev

pytestmark = pytest.mark.gpu

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_outputs.npz")
CASES = build_cases()


def gather_kernel(capi, torch, table, value_dtype, keys, *, out_dtype=None, width=0,
                  default_row=-1, hit_mask=None, out_rows_bytes=None):
    t_dev = to_dev(torch, table)
    k_dev = to_dev(torch, keys)
    raw = out_dtype is None or out_dtype == value_dtype
    if raw:
        nbytes = table.shape[1] if out_rows_bytes is None else out_rows_bytes
        out = torch.full((keys.size, nbytes), 0xAB, dtype=torch.uint8, device="cuda")
    else:
        out = torch.full((keys.size, width), 7.0,
                         dtype=torch.float32 if out_dtype == "f32" else torch.float16, device="cuda")
    g = capi.GatherArgs()
    g.table = ptr(t_dev)
    g.num_rows = table.shape[0]
    g.row_stride = table.shape[1]
    g.value_dtype = DT[value_dtype]
    g.row_width = width
    g.default_row_index = default_row
    g.cache = None
    g.key_type = capi.KEY_INT64 if keys.dtype == np.int64 else capi.KEY_INT32
    g.keys = ptr(k_dev)
    g.num_keys = keys.size
    g.output = ptr(out)
    g.output_stride = out.stride(0) * out.element_size()
    g.output_dtype = DT[value_dtype] if raw else DT[out_dtype]
    g.row_copy_bytes = out.shape[1] if raw else 0
    mask_dev = None
    if hit_mask is not None:
        mask_dev = to_dev(torch, hit_mask)
        g.hit_mask = ptr(mask_dev)
    miss = torch.zeros(1, dtype=torch.int64, device="cuda")
    g.miss_count = ptr(miss)
    capi.check(capi.lib.nve_b200_gather_rows(C.byref(g), None))
    torch.cuda.synchronize()
    return out.cpu().numpy(), (None if mask_dev is None else mask_dev.cpu().numpy()), int(miss.item())


def test_raw_gather_matches_golden(capi, torch_cuda):
    case = CASES["f16_w128_gather"]
    got, _, miss = gather_kernel(capi, torch_cuda, case["table"], "f16", case["keys"])
    assert miss == 0
    assert np.array_equal(got, GOLDEN["f16_w128_gather"])


@pytest.mark.parametrize("row_bytes", [2, 6, 20, 64, 130, 256, 260, 512, 1028, 4096])
@pytest.mark.parametrize("key_dtype", [np.int32, np.int64])
def test_raw_gather_row_sizes(capi, torch_cuda, oracle, row_bytes, key_dtype):
    rows = 500
    table = np.random.default_rng(row_bytes).integers(0, 256, (rows, row_bytes), dtype=np.uint8)
    keys = dg.uniform_keys(1237, rows, 3).astype(key_dtype)
    got, _, _ = gather_kernel(capi, torch_cuda, table, "f16", keys)
    want = np.zeros_like(got)
    oracle.gather(table, keys, want)
    assert np.array_equal(got, want)


def test_gather_hit_mask_and_misses(capi, torch_cuda, oracle):
    """Out-of-range keys stay unresolved, pre-set mask bits are skipped, the word layout is the
    little-endian 64-bit one."""
    rows, rb = 200, 64
    table = np.random.default_rng(1).integers(0, 256, (rows, rb), dtype=np.uint8)
    n = 333
    keys = dg.uniform_keys(n, rows, 2)
    keys[[3, 64, 65, 200, 332]] = [-5, 200, 1 << 40, -1, 999]
    mask = np.zeros((n + 63) // 64, dtype=np.uint64)
    pre = [0, 31, 32, 63, 64, 100, 331]
    for i in pre:
        mask[i // 64] |= np.uint64(1) << np.uint64(i % 64)
    got, got_mask, miss = gather_kernel(capi, torch_cuda, table, "f16", keys, hit_mask=mask.copy())
    want = np.full_like(got, 0xAB)
    want_mask = mask.copy()
    hits = oracle.gather(table, keys, want, want_mask)
    assert np.array_equal(got, want)
    assert np.array_equal(got_mask.view(np.uint64), want_mask)
    assert miss == n - len(pre) - hits == 4   # position 64 was pre-resolved


@pytest.mark.parametrize("name", ["qint8f16_w128_concat_f16", "f16_w96_concat_f32"])
def test_convert_gather_matches_golden(capi, torch_cuda, name):
    case = CASES[name]
    got, _, _ = gather_kernel(capi, torch_cuda, case["table"], case["value_dtype"], case["keys"],
                              out_dtype=case["out_dtype"], width=case["width"])
    assert np.array_equal(got.view(np.uint8), GOLDEN[name].view(np.uint8))


@pytest.mark.parametrize("vd", ["qint8_f32", "qint8_f16", "quint8_f32", "quint8_f16"])
def test_dequant_gather_vs_oracle(capi, torch_cuda, oracle, vd):
    for width, stride in ((256, None), (30, None), (100, 112), (1024, None)):
        table = dg.quantized_rows(400, width, 5, vd, stride=stride)
        keys = dg.uniform_keys(555, 400, 6)
        for od in ("f32", "f16"):
            got, _, _ = gather_kernel(capi, torch_cuda, table, vd, keys, out_dtype=od, width=width)
            want = oracle.lookup_pooled(table, vd, width, keys, "concat", out_dtype=od)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (width, od)


def test_layer_plain_lookup_and_default_row(capi, torch_cuda, oracle):
    torch = torch_cuda
    case = CASES["f16_w128_gather"]
    table = case["table"]
    t_dev = to_dev(torch, table)
    layer = GpuLayer(t_dev, table.shape[0], table.shape[1], "f16", default_row=17)
    keys = case["keys"].copy()
    keys[::50] = -1
    keys[1::50] = table.shape[0] + 5
    out = np.zeros((keys.size, table.shape[1]), dtype=np.uint8)
    hr = layer.lookup(keys, out, table.shape[1])
    layer.ctx.wait()
    fixed = np.where((keys < 0) | (keys >= table.shape[0]), 17, keys)
    assert hr == 1.0
    assert np.array_equal(out, table[fixed])
    layer.close()


def test_layer_quantised_raw_rows_include_metadata(capi, torch_cuda):
    torch = torch_cuda
    table = dg.quantized_rows(300, 64, 8, "quint8_f32")
    layer = GpuLayer(to_dev(torch, table), 300, table.shape[1], "quint8_f32", key_type=capi.KEY_INT32)
    keys = dg.uniform_keys(100, 300, 9).astype(np.int32)
    out = np.zeros((100, table.shape[1]), dtype=np.uint8)
    layer.lookup(keys, out, table.shape[1])
    layer.ctx.wait()
    assert np.array_equal(out, table[keys])
    layer.close()


def test_layer_update_and_accumulate_match_golden(capi, torch_cuda, oracle):
    torch = torch_cuda
    case = CASES["f32_w64_update_accumulate"]
    table = case["table"].view(np.float32).copy()
    t_dev = to_dev(torch, table)
    layer = GpuLayer(t_dev, table.shape[0], 256, "f32")
    layer.accumulate(case["keys"], case["updates"], 256, 256, "f32")   # host buffers
    layer.ctx.wait()
    got = t_dev.cpu().numpy()
    want = GOLDEN["f32_w64_update_accumulate"]
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) <= 1e-6
    assert np.array_equal(got, want)   # unique keys: one add per element, exact
    # update: overwrite rows, out-of-range keys ignored
    keys = np.array([3, 700, -1, 5], dtype=np.int64)
    vals = np.random.default_rng(3).normal(size=(4, 64)).astype(np.float32)
    layer.update(to_dev(torch, keys), to_dev(torch, vals), 256, 256)
    layer.ctx.wait()
    now = t_dev.cpu().numpy()
    want2 = want.copy()
    oracle.update(want2.view(np.uint8).reshape(512, -1), keys, vals.view(np.uint8).reshape(4, -1))
    assert np.array_equal(now, want2)
    layer.close()


@pytest.mark.parametrize("vd,npdt", [("f32", np.float32), ("f16", np.float16)])
def test_accumulate_duplicate_keys_sum(capi, torch_cuda, vd, npdt):
    """Same key many times in one call: every contribution lands (reference
    tests/kernels/update_accumulate_tests.cu:82-88).  Dyadic values make the sum order-free."""
    torch = torch_cuda
    rows, width = 64, 40
    # multiples of 1/8 below 1 in magnitude: 50 of them still sum exactly in fp16
    table = (np.round(dg.dyadic_table(rows, width, 1, np.float32) * 8) / 8).astype(npdt)
    t_dev = to_dev(torch, table)
    layer = GpuLayer(t_dev, rows, width * table.itemsize, vd)
    keys = np.array([7] * 50 + [9] * 3 + [63, -2, 64], dtype=np.int64)
    upd = (np.round(dg.dyadic_table(keys.size, width, 2, np.float32) * 8) / 8).astype(npdt)
    layer.accumulate(keys, upd, width * table.itemsize, width * table.itemsize, vd)
    layer.ctx.wait()
    want = table.astype(np.float64)
    for k, u in zip(keys, upd):
        if 0 <= k < rows:
            want[k] += u.astype(np.float64)
    assert np.array_equal(t_dev.cpu().numpy().astype(np.float64), want)
    layer.close()
