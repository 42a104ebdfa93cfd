"""Backward of a pooled lookup (nve_b200_pooling_backprop and the pynve-named edge) against the
oracle (bit-exact: same order of additions) and against the reference's GradientCalculator run on
the same GPU (tolerance 1e-6: it multiplies and adds fused, and combines split groups with
atomics)."""
import ctypes as C

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import to_dev

pytestmark = pytest.mark.gpu

POOL = {"sum": capi.POOL_SUM, "mean": capi.POOL_MEAN, "wsum": capi.POOL_WEIGHTED_SUM,
        "wmean": capi.POOL_WEIGHTED_MEAN}


def make_case(n_bags, rows, width, seed, hot_key=True):
    rng = np.random.default_rng(seed)
    lens = rng.integers(1, 33, n_bags)
    csr = np.zeros(n_bags + 1, np.int64)
    csr[1:] = np.cumsum(lens)
    n = int(csr[-1])
    keys = dg.zipf_keys(n, rows, 1.05, seed + 1, dg.permutation(rows))
    if hot_key:
        keys[::3] = keys[1]                       # one key far beyond 1024 occurrences: split group
    grads = rng.normal(0, 1e-2, (n_bags, width)).astype(np.float32)
    weights = rng.uniform(0.25, 2.0, n).astype(np.float32)
    return keys, csr, grads, weights


def run_mine(torch, keys, csr, grads, weights, pooling, max_run=1024, fixed_hot=0):
    n, width = keys.size, grads.shape[1]
    d = C.c_void_p()
    capi.check(capi.lib.nve_b200_deduper_create(C.byref(d), capi.KEY_INT64, max_run, n))
    k, g = to_dev(torch, keys), to_dev(torch, grads)
    o = to_dev(torch, csr) if csr is not None else None
    w = to_dev(torch, weights) if weights is not None else None
    uniq = torch.full((n,), -1, dtype=torch.int64, device="cuda")
    out = torch.full((n, width), 7.0, device="cuda")
    nu = C.c_int64(0)
    for _ in range(2):                            # twice: scratch is reused
        capi.check(capi.lib.nve_b200_pooling_backprop(
            d, n, k.data_ptr(), g.data_ptr(), width * 4, width * 4, POOL[pooling],
            capi.SPARSE_CSR if csr is not None else capi.SPARSE_FIXED, o.data_ptr() if o is not None else None,
            grads.shape[0], fixed_hot, w.data_ptr() if w is not None else None, uniq.data_ptr(),
            out.data_ptr(), width * 4, C.byref(nu), None))
    capi.check(capi.lib.nve_b200_deduper_destroy(d))
    u = nu.value
    return uniq[:u].cpu().numpy(), out[:u].cpu().numpy()


@pytest.mark.parametrize("pooling", ["sum", "mean", "wsum", "wmean"])
@pytest.mark.parametrize("width", [32, 128, 212])
def test_matches_oracle_bit_for_bit(torch_cuda, oracle, pooling, width):
    keys, csr, grads, weights = make_case(1500, 2500, width, 3)
    w = weights if pooling in ("wsum", "wmean") else None
    uniq, got = run_mine(torch_cuda, keys, csr, grads, w, pooling)
    want_u, want = oracle.pooling_backprop(keys, csr, grads, pooling, w)
    assert np.array_equal(uniq, want_u)
    assert np.array_equal(got, want)
    # against exact arithmetic
    lens = np.diff(csr)
    bag = np.repeat(np.arange(lens.size), lens)
    ww = np.ones(keys.size) if w is None else w.astype(np.float64)
    if pooling in ("mean", "wmean"):
        sums = np.add.reduceat(ww, csr[:-1])
        ww = ww / sums[bag]
    exact = np.zeros((uniq.size, width))
    np.add.at(exact, np.searchsorted(uniq, keys), ww[:, None] * grads.astype(np.float64)[bag])
    assert np.max(np.abs(got - exact)) <= 1e-6 * max(1.0, np.abs(exact).max()) * 8


def test_fixed_hotness_and_no_splitting(torch_cuda, oracle):
    rows, width, bags, hot = 900, 64, 700, 8
    keys = dg.zipf_keys(bags * hot, rows, 1.1, 11, dg.permutation(rows))
    grads = np.random.default_rng(12).normal(0, 1e-2, (bags, width)).astype(np.float32)
    csr = np.arange(0, bags * hot + 1, hot, dtype=np.int64)
    uniq, got = run_mine(torch_cuda, keys, None, grads, None, "mean", max_run=-1, fixed_hot=hot)
    want_u, want = oracle.pooling_backprop(keys, csr, grads, "mean", None, max_run=-1)
    assert np.array_equal(uniq, want_u) and np.array_equal(got, want)


@pytest.mark.parametrize("pooling", ["sum", "wsum", "wmean"])
def test_matches_reference_gpu(torch_cuda, reference_gpu, pooling):
    torch = torch_cuda
    width = 128
    keys, csr, grads, weights = make_case(2000, 3000, width, 5)
    n = keys.size
    w = weights if pooling != "sum" else None
    uniq, got = run_mine(torch, keys, csr, grads, w, pooling)
    k, o, g = to_dev(torch, keys), to_dev(torch, csr), to_dev(torch, grads)
    wd = to_dev(torch, weights)
    r_uniq = torch.full((n,), -1, dtype=torch.int64, device="cuda")
    r_out = torch.zeros((n, width), device="cuda")
    u = reference_gpu.pooling_backprop(k.data_ptr(), n, o.data_ptr(), csr.size - 1, g.data_ptr(),
                                       wd.data_ptr() if w is not None else None, pooling, width,
                                       r_uniq.data_ptr(), r_out.data_ptr())
    assert u == uniq.size
    assert np.array_equal(r_uniq[:u].cpu().numpy(), uniq)
    want = r_out[:u].cpu().numpy()
    assert np.max(np.abs(got - want)) <= 1e-6 * max(1.0, float(np.abs(want).max())) * 8


def test_pynve_edge(torch_cuda, oracle):
    torch = torch_cuda
    from nv_embedding_cache_b200 import pynve
    rows, width = 4000, 64
    table = torch.zeros((rows, width), device="cuda")
    layer = pynve.GPUEmbedding(width, rows, pynve.DataType_t.Float32, table, 0)
    keys, csr, grads, weights = make_case(800, rows, width, 21, hot_key=False)
    n = keys.size
    k, o, g, w = to_dev(torch, keys), to_dev(torch, csr), to_dev(torch, grads), to_dev(torch, weights)
    uniq = torch.empty(n, dtype=torch.int64, device="cuda")
    out = torch.empty((n, width), device="cuda")
    u = layer.pooling_backprop(n, k.data_ptr(), g.data_ptr(), uniq.data_ptr(), out.data_ptr(),
                               int(pynve.PoolingType_t.WeightedSum), csr.size - 1, o.data_ptr(),
                               int(pynve.DataType_t.Float32), w.data_ptr(), 0)
    want_u, want = oracle.pooling_backprop(keys, csr, grads, "wsum", weights)
    assert u == want_u.size
    assert np.array_equal(uniq[:u].cpu().numpy(), want_u)
    assert np.array_equal(out[:u].cpu().numpy(), want)
    layer.close()
