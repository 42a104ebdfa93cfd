"""Regenerates tests/golden/reference_outputs.npz by running the UNMODIFIED reference CPU path
(oracle/_ref/libnve_ref.so, built from the reference checkout by oracle/build.py) on the seeded
cases of cases.py.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from golden.cases import build_cases  # noqa: E402
from oracle.pyoracle import NP_OF, DT, Reference  # noqa: E402


def run_reference(ref: Reference, case: dict) -> np.ndarray:
    table = case["table"].copy()
    layer = ref.layer(table, case["value_dtype"])
    try:
        if case["op"] == "gather":
            out = np.zeros((case["keys"].size, table.shape[1]), dtype=np.uint8)
            layer.lookup(case["keys"], out)
            return out
        if case["op"] == "accumulate":
            layer.accumulate(case["keys"], case["updates"])
            return table.view(np.float32).copy()
        return layer.lookup_pooled(case["keys"], case["pooling"], case["width"],
                                   offsets=case["offsets"], hotness=case["hotness"],
                                   weights=case["weights"], out_dtype=case["out_dtype"])
    finally:
        layer.close()


def main():
    ref = Reference()
    outs = {}
    for name, case in build_cases().items():
        outs[name] = run_reference(ref, case)
        print(f"{name}: {outs[name].shape} {outs[name].dtype}")
    np.savez_compressed(Path(__file__).resolve().parent / "reference_outputs.npz", **outs)


if __name__ == "__main__":
    main()
