"""The device-side cache contract for user kernels (include/nve_b200_ecache.cuh): a kernel written
against CacheData + AddressFunctor::get_address, compiled here with nvcc outside the library, must
find exactly the keys the library's own lookup finds and read the same rows."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
SRC = ROOT / "tests" / "user_kernel" / "probe_kernel.cu"
NVCC = "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", f"-I{ROOT / 'include'}"]


def test_user_kernel_compiles_against_the_public_headers(tmp_path):
    obj = tmp_path / "probe_kernel.o"
    res = subprocess.run([NVCC, *ARCH, "-c", str(SRC), "-o", str(obj)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert obj.stat().st_size > 0


@pytest.mark.gpu
@pytest.mark.parametrize("key_dtype", [np.int64, np.int32])
def test_user_kernel_reads_what_the_library_reads(torch_cuda, tmp_path, key_dtype):
    torch = torch_cuda
    from nv_embedding_cache_b200 import capi, datagen as dg
    from nve_helpers import CacheTable, to_dev
    lib_path = tmp_path / "libprobe.so"
    subprocess.run([NVCC, *ARCH, "-shared", "-Xcompiler", "-fPIC", str(SRC), "-o", str(lib_path)], check=True)
    user = C.CDLL(str(lib_path))
    rows, width = 5000, 32
    rb = width * 4
    table = np.random.default_rng(3).normal(0, 1, (rows, width)).astype(np.float32)
    t_dev = to_dev(torch, table)
    kb = np.dtype(key_dtype).itemsize
    ct = CacheTable(48 * (8 * kb + 8 * rb + 32), rb, value_dtype="f32", key_dtype=key_dtype, backing=t_dev,
                    backing_rows=rows)
    warm = dg.zipf_keys(2000, rows, 1.1, 5, dg.permutation(rows))
    cached_rows = table[warm] + 100.0                     # the cache holds rows the table does not
    ct.insert(warm, cached_rows.view(np.uint8).reshape(warm.size, rb))
    keys = dg.zipf_keys(3001, rows, 1.1, 6, dg.permutation(rows)).astype(key_dtype)
    k_dev = to_dev(torch, keys)

    # the library's lookup of the same keys: rows and miss count
    out = np.zeros((keys.size, rb), np.uint8)
    lib_misses = ct.find(keys, out)
    want = out.view(np.float32).reshape(keys.size, width)[:, 0]

    view = capi.CacheData()
    ct.table.reset_lookup_counter(ct.ctx)
    capi.check(capi.lib.nve_b200_gpu_table_get_cache_data(ct.table.handle, ct.ctx.handle, C.byref(view)))
    values = torch.zeros(keys.size, dtype=torch.float32, device="cuda")
    where = torch.zeros(keys.size, dtype=torch.int32, device="cuda")
    stream = C.c_void_p()
    capi.check(capi.lib.nve_context_get_lookup_stream(ct.ctx.handle, C.byref(stream)))
    user.user_first_values.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.POINTER(capi.CacheData),
                                       C.c_void_p, C.c_void_p, C.c_void_p]
    assert user.user_first_values(kb, k_dev.data_ptr(), keys.size, t_dev.data_ptr(), C.byref(view),
                                  values.data_ptr(), where.data_ptr(), stream) == 0
    ct.ctx.wait()
    torch.cuda.synchronize()
    got = values.cpu().numpy()
    assert np.array_equal(got, want)
    from_cache = where.cpu().numpy().astype(bool)
    assert np.array_equal(from_cache, want > 50.0)        # cached rows carry the +100 marker
    assert 0 < from_cache.sum() < keys.size
    assert ct.table_counter() == lib_misses == int((~from_cache).sum())
    ct.close()
