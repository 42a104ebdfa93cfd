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


TORCH_OPS_SRC = CSRC / "torch" / "nve_torch_ops.cpp"
TORCH_OPS_LIB = PKG / "libnve_b200_torch_ops.so"


def build_torch_ops(force: bool = False, verbose: bool = False) -> Path | None:
    """Builds libnve_b200_torch_ops.so (the torch custom ops over the layer registry) with the host
    compiler against the installed torch's stable-ABI headers.  Returns None when torch is not
    importable; the rest of the library does not need it."""
    try:
        import torch
    except ImportError:
        return None
    build()
    torch_dir = Path(torch.__file__).resolve().parent
    newest = max(TORCH_OPS_SRC.stat().st_mtime, (ROOT / "include" / "nve_b200_ops.h").stat().st_mtime)
    if not force and TORCH_OPS_LIB.exists() and TORCH_OPS_LIB.stat().st_mtime >= newest:
        return TORCH_OPS_LIB
    cuda_include = Path(NVCC).resolve().parent.parent / "include"
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-I{torch_dir / 'include'}", f"-I{cuda_include}", f"-I{ROOT / 'include'}", str(TORCH_OPS_SRC),
           "-o", str(TORCH_OPS_LIB), f"-L{PKG}", "-lnve_b200", "-Wl,-rpath,$ORIGIN",
           f"-L{torch_dir / 'lib'}", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{torch_dir / 'lib'}"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return TORCH_OPS_LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--bounds-check", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.bounds_check))
    if not a.bounds_check:
        print(build_torch_ops(a.force, a.verbose))
    sys.exit(0)
