"""Builds libnve_b200.so (the C-ABI library of the lookup hot path) in-tree with nvcc for sm_100a.

    python -m nv_embedding_cache_b200.build [--force] [--verbose] [--bounds-check]

Objects go to ``nv_embedding_cache_b200/build/`` (git-ignored), the shared library next to this
file.  Each translation unit is compiled by its own nvcc process, several at a time.

``--bounds-check`` builds ``libnve_b200_checked.so`` instead (objects in ``build_checked/``): the same
library with -DNVE_B200_BOUNDS_CHECK, whose pooled kernels test CSR offsets and keys instead of
trusting them and report at ``nve_context_wait``.  ``NVE_B200_LIBRARY=<path>`` makes the Python
binding load it.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libnve_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden", f"-I{ROOT / 'include'}", f"-I{CSRC}"]


def sources():
    return sorted(CSRC.rglob("*.cu"))


def _deps_mtime() -> float:
    hdrs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) + list((ROOT / "include").glob("*.h"))
    return max(p.stat().st_mtime for p in hdrs)


LIB_CHECKED = PKG / "libnve_b200_checked.so"
OBJ_CHECKED = PKG / "build_checked"


def _compile(src: Path, force: bool, verbose: bool, hdr_mtime: float, obj_dir: Path = OBJ, extra=()) -> Path:
    obj = obj_dir / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
    if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_mtime):
        return obj
    cmd = [NVCC, *ARCH, *FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, bounds_check: bool = False) -> Path:
    obj_dir, lib = (OBJ_CHECKED, LIB_CHECKED) if bounds_check else (OBJ, LIB)
    extra = ("-DNVE_B200_BOUNDS_CHECK",) if bounds_check else ()
    obj_dir.mkdir(exist_ok=True)
    srcs = sources()
    hdr_mtime = _deps_mtime()
    jobs = max(1, min(len(srcs), (os.cpu_count() or 2)))
    with ThreadPoolExecutor(jobs) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose, hdr_mtime, obj_dir, extra), srcs))
    if (not force and lib.exists()
            and lib.stat().st_mtime >= max(o.stat().st_mtime for o in objs)):
        return lib
    cmd = [NVCC, *ARCH, "-shared", "-o", str(lib), *map(str, objs), "-lpthread", "-ldl"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--bounds-check", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.bounds_check))
    sys.exit(0)
