"""The allocation-free gradient reduction (nve_b200_dedup_grads_static) against the regular entry
point (nve_b200_dedup_grads), through the C ABI.

Who needs it: code that reduces gradients where it may not allocate device memory -- inside a
training step whose memory pool is already fully planned, in a plugin that owns only the buffers it
was handed, or on a thread that must not enter the driver's allocator.  Its scratch is a 4 MiB array
built into the library, shared by all calls, so the checks run two calls in a row (the second sees
the first one's leftovers) and compare bit for bit: both entry points add in the same order.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test."""
import ctypes as C

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import ptr, to_dev

pytestmark = pytest.mark.gpu


def run_both(torch, keys, grads, max_run, fused_table=None, alpha=1.0):
    n, width = grads.shape
    d = C.c_void_p()
    capi.check(capi.lib.nve_b200_deduper_create(C.byref(d), capi.KEY_INT64, max_run, n))
    cap = n + (n // max_run if max_run > 0 else 0) + 2
    i64 = dict(dtype=torch.int64, device="cuda")
    uniq, counts, inverse = torch.zeros(n + 1, **i64), torch.zeros(n + 1, **i64), torch.zeros(n + 1, **i64)
    offsets, loc = torch.zeros(cap + 1, **i64), torch.zeros(cap + 1, **i64)
    d_keys, d_grads = to_dev(torch, keys), to_dev(torch, grads)
    runs = (C.c_int64 * 2)()
    capi.check(capi.lib.nve_b200_deduper_dedup(d, ptr(d_keys), n, ptr(uniq), ptr(counts), ptr(loc), runs,
                                               ptr(inverse), ptr(offsets), None, 0))
    u = int(runs[0])
    num_runs_dev = C.c_void_p()
    capi.check(capi.lib.nve_b200_deduper_device_num_runs(d, C.byref(num_runs_dev)))
    if fused_table is None:
        dst_a = torch.full((u, width), 5.0, device="cuda")
        dst_b = torch.full((u, width), -5.0, device="cuda")
        fused, rows = 0, 0
    else:
        dst_a, dst_b = to_dev(torch, fused_table), to_dev(torch, fused_table)
        fused, rows = 1, fused_table.shape[0]
    capi.check(capi.lib.nve_b200_dedup_grads(d, ptr(d_grads), width * 4, width * 4, n, ptr(uniq), ptr(inverse),
                                             ptr(offsets), ptr(loc), ptr(dst_a), width * 4, fused, rows,
                                             alpha, None))
    capi.check(capi.lib.nve_b200_dedup_grads_static(
        capi.KEY_INT64, max_run, ptr(d_grads), width * 4, width * 4, n, ptr(uniq), ptr(inverse),
        ptr(offsets), ptr(loc), num_runs_dev, ptr(dst_b), width * 4, fused, rows, alpha, None))
    torch.cuda.synchronize()
    a, b = dst_a.cpu().numpy(), dst_b.cpu().numpy()
    capi.check(capi.lib.nve_b200_deduper_destroy(d))
    return a, b, u


def test_static_scratch_matches_regular_entry_point_twice(torch_cuda):
    torch = torch_cuda
    rows, width = 3000, 128
    for call, (seed, n) in enumerate([(1, 40000), (2, 25000)]):     # two calls in a row
        keys = dg.zipf_keys(n, rows, 1.05, seed, dg.permutation(rows))
        keys[::5] = keys[0]                       # a group far longer than one chunk: uses the scratch
        grads = np.random.default_rng(seed).normal(0, 1e-2, (n, width)).astype(np.float32)
        a, b, u = run_both(torch, keys, grads, max_run=1024)
        assert u == np.unique(keys).size
        assert np.array_equal(a, b), f"call {call}"
        want = np.zeros((u, width), np.float64)
        np.add.at(want, np.searchsorted(np.unique(keys), keys), grads.astype(np.float64))
        assert np.max(np.abs(b - want)) <= 1e-6 * 50 * max(1.0, np.abs(want).max())


def test_static_fused_apply_and_unsplit_runs(torch_cuda):
    torch = torch_cuda
    rows, width, n = 2000, 64, 30000
    table = dg.normal_table(rows, width, 0.02, 3, np.float32)
    keys = dg.zipf_keys(n, rows, 1.05, 4, dg.permutation(rows))
    grads = np.random.default_rng(5).normal(0, 1e-2, (n, width)).astype(np.float32)
    for max_run in (1024, 64, -1):
        a, b, _ = run_both(torch, keys, grads, max_run=max_run, fused_table=table, alpha=-0.01)
        assert np.array_equal(a, b), max_run
        assert not np.array_equal(b, table)


def test_static_rejects_more_than_its_scratch(torch_cuda):
    # 1M keys in runs of 16 with 512-byte rows would need ~64 MiB of partial sums
    st = capi.lib.nve_b200_dedup_grads_static(capi.KEY_INT64, 16, 1, 512, 512, 1 << 20, 1, 1, 1, 1, 1, 1,
                                              512, 0, 0, 1.0, None)
    assert st == capi.NVE_ERROR_INVALID_ARGUMENT
    msg = capi.last_error()
    assert "built-in scratch holds 4194304" in msg and "nve_b200_dedup_grads" in msg
