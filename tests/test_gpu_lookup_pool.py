"""GPU parity of the fused lookup+pool kernel and the dense-table layer, through the C ABI,
against the committed golden vectors (reference CPU outputs) and the C oracle."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from golden.cases import build_cases
from nv_embedding_cache_b200 import datagen as dg
from nve_helpers import DT, POOL, GpuLayer, ptr, rel_err, to_dev

pytestmark = pytest.mark.gpu

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_outputs.npz")
CASES = build_cases()
POOLED = sorted(n for n, c in CASES.items() if c["op"] == "pooled" and c["pooling"] != "concat")
CONCAT = sorted(n for n, c in CASES.items() if c["op"] == "pooled" and c["pooling"] == "concat")


def run_pool_kernel(capi, torch, case, *, key_dtype=np.int64, off_dtype=np.int64, out=None,
                    default_row=-1, table_dev=None, gathered=False):
    table = case["table"]
    if gathered:            # rows already gathered in key order: pooled with keys == NULL
        table = np.ascontiguousarray(table[case["keys"]])
    t_dev = to_dev(torch, table) if table_dev is None else table_dev
    keys = to_dev(torch, case["keys"].astype(key_dtype))
    offs = None if case["offsets"] is None else to_dev(torch, case["offsets"].astype(off_dtype))
    w = None if case["weights"] is None else to_dev(torch, case["weights"])
    nbags = (case["offsets"].size - 1) if case["offsets"] is not None else case["keys"].size // case["hotness"]
    np_out = np.float32 if case["out_dtype"] == "f32" else np.float16
    if out is None:
        out = torch.full((nbags, case["width"]), 7.0,
                         dtype=torch.float32 if np_out == np.float32 else torch.float16, device="cuda")
    a = capi.PoolArgs()
    a.table = ptr(t_dev)
    a.num_rows = table.shape[0]
    a.row_stride = table.shape[1]
    a.value_dtype = DT[case["value_dtype"]]
    a.row_width = case["width"]
    a.default_row_index = default_row
    a.cache = None
    a.key_type = capi.KEY_INT64 if key_dtype == np.int64 else capi.KEY_INT32
    a.keys = None if gathered else ptr(keys)
    a.num_keys = case["keys"].size
    a.pooling_type = POOL[case["pooling"]]
    a.sparse_type = capi.SPARSE_CSR if offs is not None else capi.SPARSE_FIXED
    a.csr_offsets = ptr(offs)
    a.offset_bytes = np.dtype(off_dtype).itemsize
    a.num_bags = nbags
    a.fixed_hotness = case["hotness"]
    a.weights = ptr(w)
    a.weight_dtype = 0 if case["weights"] is None else (
        capi.DTYPE_FLOAT32 if case["weights"].dtype == np.float32 else capi.DTYPE_FLOAT16)
    a.output = ptr(out)
    a.output_stride = out.stride(0) * out.element_size()
    a.output_dtype = DT[case["out_dtype"]]
    capi.check(capi.lib.nve_b200_lookup_pool(C.byref(a), None))
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("name", POOLED)
def test_kernel_matches_golden_bit_for_bit(capi, torch_cuda, name):
    """Accumulation order and rounding follow the scalar reference, so even weighted / mean /
    dequantised results are identical, not merely within 1e-5."""
    got = run_pool_kernel(capi, torch_cuda, CASES[name])
    want = GOLDEN[name]
    assert rel_err(got, want) <= 1e-5  # the stated tolerance
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("name", POOLED)
def test_pooling_of_gathered_rows(capi, torch_cuda, name):
    """keys == NULL pools rows that an earlier step gathered (the last step of a multi-tier lookup,
    the reference's pool_gathered_device): same bits as the fused lookup."""
    got = run_pool_kernel(capi, torch_cuda, CASES[name], gathered=True)
    assert np.array_equal(got.view(np.uint8), GOLDEN[name].view(np.uint8))
    got = run_pool_kernel(capi, torch_cuda, CASES[name], gathered=True, key_dtype=np.int32, off_dtype=np.int32)
    assert np.array_equal(got.view(np.uint8), GOLDEN[name].view(np.uint8))


@pytest.mark.parametrize("name", POOLED[:6])
def test_kernel_int32_keys_and_offsets(capi, torch_cuda, name):
    got = run_pool_kernel(capi, torch_cuda, CASES[name], key_dtype=np.int32, off_dtype=np.int32)
    assert np.array_equal(got.view(np.uint8), GOLDEN[name].view(np.uint8))
    got = run_pool_kernel(capi, torch_cuda, CASES[name], key_dtype=np.int64, off_dtype=np.int32)
    assert np.array_equal(got.view(np.uint8), GOLDEN[name].view(np.uint8))


def test_kernel_unaligned_table_and_output(capi, torch_cuda, oracle):
    """Base pointers that are only element-aligned force the narrow-vector variants."""
    torch = torch_cuda
    case = dict(CASES["f16_w128_csr_mean"])
    raw = case["table"]
    buf = torch.zeros(raw.size + 64, dtype=torch.uint8, device="cuda")
    for shift in (2, 4, 8):
        view = buf[shift:shift + raw.size].view(raw.shape[0], raw.shape[1])
        view.copy_(torch.from_numpy(raw))
        got = run_pool_kernel(capi, torch, case, table_dev=view)
        assert np.array_equal(got.view(np.uint8), GOLDEN["f16_w128_csr_mean"].view(np.uint8))
    nbags = case["offsets"].size - 1
    obuf = torch.zeros(nbags * 128 + 8, dtype=torch.float16, device="cuda")
    out = obuf[1:1 + nbags * 128].view(nbags, 128)
    got = run_pool_kernel(capi, torch, case, out=out)
    assert np.array_equal(got.view(np.uint8), GOLDEN["f16_w128_csr_mean"].view(np.uint8))


@pytest.mark.parametrize("vd,width,stride", [("qint8_f32", 256, 272), ("quint8_f16", 30, 48),
                                             ("qint8_f16", 1000, 1002), ("quint8_f32", 2048, 2056)])
def test_kernel_quantised_padded_and_wide_rows(capi, torch_cuda, oracle, vd, width, stride):
    """Padded strides (legal for the device kernel, not expressible through the host layer) and
    rows wider than one pass of a warp, against the C oracle."""
    rows = 900
    table = dg.quantized_rows(rows, width, 77, vd, stride=stride)
    _, offs = dg.csr_bags(50, 0, 70, 78)
    keys = dg.uniform_keys(int(offs[-1]), rows, 79)
    w = np.random.default_rng(80).uniform(-1, 1, keys.size).astype(np.float32)
    for pooling in ("sum", "wmean"):
        for od in ("f32", "f16"):
            case = dict(table=table, value_dtype=vd, width=width, keys=keys, offsets=offs,
                        hotness=0, weights=w if pooling == "wmean" else None, pooling=pooling,
                        out_dtype=od)
            got = run_pool_kernel(capi, torch_cuda, case)
            want = oracle.lookup_pooled(table, vd, width, keys, pooling, offsets=offs,
                                        weights=case["weights"], out_dtype=od)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (pooling, od)


@pytest.mark.parametrize("width", [1, 2, 3, 7, 64, 132, 1024, 3000])
@pytest.mark.parametrize("vd", ["f32", "f16"])
def test_kernel_width_sweep(capi, torch_cuda, oracle, vd, width):
    rows = 300
    npdt = np.float32 if vd == "f32" else np.float16
    t = dg.dyadic_table(rows, width, width, npdt)
    table = t.view(np.uint8).reshape(rows, -1)
    for hot in (1, 31, 32, 33, 100):
        keys = dg.uniform_keys(hot * 9, rows, hot)
        case = dict(table=table, value_dtype=vd, width=width, keys=keys, offsets=None, hotness=hot,
                    weights=None, pooling="sum", out_dtype=vd)
        got = run_pool_kernel(capi, torch_cuda, case)
        want = oracle.lookup_pooled(table, vd, width, keys, "sum", hotness=hot, out_dtype=vd)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), hot


def test_kernel_default_row_and_empty_bags(capi, torch_cuda, oracle):
    rows, width = 100, 64
    t = dg.dyadic_table(rows, width, 5, np.float32)
    table = t.view(np.uint8).reshape(rows, -1)
    keys = np.array([5, -3, 1000, 7, 99, 100, 0], dtype=np.int64)
    offs = np.array([0, 0, 3, 3, 7, 7], dtype=np.int64)
    case = dict(table=table, value_dtype="f32", width=width, keys=keys, offsets=offs, hotness=0,
                weights=None, pooling="mean", out_dtype="f32")
    got = run_pool_kernel(capi, torch_cuda, case, default_row=42)
    want = oracle.lookup_pooled(table, "f32", width, keys, "mean", offsets=offs, default_row=42)
    assert np.array_equal(got, want)
    assert not got[0].any() and not got[2].any() and not got[4].any()


def test_kernel_zero_weight_sum_gives_zero_row(capi, torch_cuda, oracle):
    rows, width = 50, 32
    t = dg.dyadic_table(rows, width, 6, np.float32)
    table = t.view(np.uint8).reshape(rows, -1)
    keys = np.array([1, 2, 3, 4], dtype=np.int64)
    w = np.array([0.5, -0.5, 0.25, 0.25], dtype=np.float32)
    case = dict(table=table, value_dtype="f32", width=width, keys=keys, offsets=None, hotness=2,
                weights=w, pooling="wmean", out_dtype="f32")
    got = run_pool_kernel(capi, torch_cuda, case)
    want = oracle.lookup_pooled(table, "f32", width, keys, "wmean", hotness=2, weights=w)
    assert np.array_equal(got, want)
    assert not got[0].any()


# ---- layer level (nve_layer_lookup_pooled) ----------------------------------------------------
LAYER_LEGAL = [n for n in POOLED if (
    CASES[n]["value_dtype"] == CASES[n]["out_dtype"] or
    CASES[n]["value_dtype"].endswith(CASES[n]["out_dtype"]))
    and (CASES[n]["weights"] is None or not CASES[n]["value_dtype"].startswith("f")
         or CASES[n]["weights"].dtype == (np.float32 if CASES[n]["value_dtype"] == "f32" else np.float16))]


@pytest.mark.parametrize("name", LAYER_LEGAL)
@pytest.mark.parametrize("host_buffers", [False, True])
def test_layer_lookup_pooled_matches_golden(capi, torch_cuda, name, host_buffers):
    torch = torch_cuda
    case = CASES[name]
    t_dev = to_dev(torch, case["table"])
    layer = GpuLayer(t_dev, case["table"].shape[0], case["table"].shape[1], case["value_dtype"])
    want = GOLDEN[name]
    wd = "f32" if case["weights"] is None or case["weights"].dtype == np.float32 else "f16"
    if host_buffers:
        out = np.zeros_like(want)
        hr = layer.lookup_pooled(case["keys"], out, out.strides[0], case["pooling"],
                                 offsets=case["offsets"], hotness=case["hotness"],
                                 weights=case["weights"], weight_dtype=wd, out_dtype=case["out_dtype"])
        layer.ctx.wait()
        got = out
    else:
        keys = to_dev(torch, case["keys"])
        offs = None if case["offsets"] is None else to_dev(torch, case["offsets"])
        w = None if case["weights"] is None else to_dev(torch, case["weights"])
        out = torch.zeros(want.shape, dtype=torch.float32 if want.dtype == np.float32 else torch.float16,
                          device="cuda")
        hr = layer.lookup_pooled(keys, out, out.stride(0) * out.element_size(), case["pooling"],
                                 offsets=offs, hotness=case["hotness"], weights=w, weight_dtype=wd,
                                 out_dtype=case["out_dtype"])
        layer.ctx.wait()
        got = out.cpu().numpy()
    assert hr == 1.0
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
    layer.close()


def test_layer_rejects_what_the_reference_rejects(capi, torch_cuda):
    torch = torch_cuda
    case = CASES["f16_w128_csr_mean"]
    t_dev = to_dev(torch, case["table"])
    layer = GpuLayer(t_dev, 5000, 256, "f16")
    keys = to_dev(torch, case["keys"])
    offs = to_dev(torch, case["offsets"])
    out = torch.zeros((300, 128), dtype=torch.float16, device="cuda")
    mask = torch.zeros(64, dtype=torch.int64, device="cuda")

    def status(fn):
        try:
            fn()
        except capi.NveError as e:
            return e.status
        return 0

    INV = capi.NVE_ERROR_INVALID_ARGUMENT
    # cross-precision output, wrong stride, missing weights, bad hotness, unknown output type
    assert status(lambda: layer.lookup_pooled(keys, out, 256, "mean", offsets=offs, out_dtype="f32")) == INV
    assert status(lambda: layer.lookup_pooled(keys, out, 512, "mean", offsets=offs, out_dtype="f16")) == INV
    assert status(lambda: layer.lookup_pooled(keys, out, 256, "wsum", offsets=offs, out_dtype="f16")) == INV
    assert status(lambda: layer.lookup_pooled(keys, out, 256, "sum", hotness=0, out_dtype="f16")) == INV
    assert status(lambda: layer.lookup_pooled(keys, out, 256, "sum", hotness=7, out_dtype="f16")) == INV
    st = capi.lib.nve_layer_lookup_pooled(layer.h, layer.ctx.h, keys.numel(), ptr(keys), ptr(out), 256,
                                          None, capi.POOL_SUM, capi.SPARSE_CSR, ptr(offs), 301, 0, None,
                                          0, capi.DTYPE_UNKNOWN, None)
    assert st == INV
    # hitmask is not supported by the dense layer
    st = capi.lib.nve_layer_lookup(layer.h, layer.ctx.h, 10, ptr(keys), ptr(out), 256, ptr(mask), None)
    assert st == INV and "Hitmask" in capi.last_error()
    # weights of another type than the table
    w32 = torch.ones(keys.numel(), dtype=torch.float32, device="cuda")
    assert status(lambda: layer.lookup_pooled(keys, out, 256, "wsum", offsets=offs, weights=w32,
                                              weight_dtype="f32", out_dtype="f16")) == INV
    layer.close()


def test_layer_empty_lookup_zero_fills_csr_bags(capi, torch_cuda):
    torch = torch_cuda
    t = dg.dyadic_table(64, 32, 1, np.float32)
    t_dev = to_dev(torch, t)
    layer = GpuLayer(t_dev, 64, 128, "f32")
    keys = torch.zeros(1, dtype=torch.int64, device="cuda")
    offs = torch.zeros(5, dtype=torch.int64, device="cuda")
    out = torch.full((4, 32), 3.0, device="cuda")
    layer.lookup_pooled(keys, out, 128, "sum", offsets=offs, out_dtype="f32", num_keys=0)
    layer.ctx.wait()
    assert not out.cpu().numpy().any()
    layer.close()
