"""The benchmark's reference arm runs on host cores only, so its output contract can be checked
without a GPU: one JSON line with the reference's CPU implementation timed on the workload both arms
share, `impl` = "reference", a `cpu_baseline` that describes the run and an `e2e` object without
copies.  The other arm's line is produced on a GPU; its `config` comes from the same function."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

from oracle import build as oracle_build

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_contract_line():
    if not (oracle_build.OUT / "libnve_ref.so").exists() and not oracle_build.REFERENCE.exists():
        pytest.skip("neither the reference checkout nor its prebuilt CPU library is on this machine")
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "3"],
                         capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 3
    assert d["metric"] == "embedding keys/sec (find-and-combine)" and d["unit"] == "keys/s"
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["data"] == "synthetic"
    assert d["value"] > 0 and d["ms_per_step"] > 0
    cb = d["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "keys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # both arms describe the workload with the same function
    sys.path.insert(0, str(ROOT))
    import bench
    assert d["config"] == bench.bench_config(1)
    assert "workload" in d["config"] and "model" not in d["config"]
