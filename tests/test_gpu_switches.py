"""The library's tuning switches are environment variables read once per process, so the paths they
select (the general pooled kernel instead of the lean one, the bulk-copy gather, the register form
of the gradient reduction, other numbers of rows in flight, host-side key checks) are exercised by
running parts of this suite again in child processes under each of them."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent

CASES = [
    ("NVE_B200_NO_DENSE", "1", "test_gpu_lookup_pool.py", ""),
    ("NVE_B200_DENSE_U", "2", "test_gpu_lookup_pool.py", "kernel"),
    ("NVE_B200_DENSE_U", "16", "test_gpu_lookup_pool.py", "kernel"),
    ("NVE_B200_POOL_BLOCK", "128", "test_gpu_lookup_pool.py", "kernel"),
    ("NVE_B200_GATHER_BULK", "1", "test_gpu_gather_update.py", ""),
    ("NVE_B200_NO_GRAD_STREAM", "1", "test_gpu_dedup.py", "grad_sums or fused"),
    ("NVE_B200_GRAD_OVERLAP", "0", "test_gpu_dedup.py", "grad_sums or fused"),
    ("NVE_B200_SHARD_U", "4", "test_gpu_sharded_object.py", "peer"),
    ("NVE_B200_CHECK_KEYS", "1", "test_gpu_lookup_pool.py", "layer"),
]


@pytest.mark.parametrize("name,value,test_file,select", CASES, ids=[f"{c[0]}={c[1]}" for c in CASES])
def test_suite_part_under_switch(torch_cuda, name, value, test_file, select):
    if os.environ.get(name) == value:
        pytest.skip("already running under this switch")
    cmd = [sys.executable, "-m", "pytest", str(HERE / test_file), "-q", "-m", "gpu", "-p", "no:cacheprovider"]
    if select:
        cmd += ["-k", select]
    res = subprocess.run(cmd, env=dict(os.environ, **{name: value}), capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-1000:]
    assert " passed" in res.stdout and " failed" not in res.stdout
