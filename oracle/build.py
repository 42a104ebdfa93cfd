"""Build recipe for the parity checker (test infrastructure, not the product).

Four artefacts, all written under ``oracle/_ref/`` (git-ignored, shipped to the GPU box as built):

* ``libnve_oracle.so``  – the plain-C restatement in ``oracle/nve_oracle.c`` (always built).
* ``libnve_ref.so``     – the UNMODIFIED reference CPU path (HostEmbeddingLayer, LinearHostTable,
  cpu_ops) compiled straight from the reference checkout, wrapped by ``oracle/ref_driver.cpp``.
  Built only where the reference checkout is present; elsewhere the prebuilt file is used.
* ``libnve_ref_gpu.so`` – the UNMODIFIED reference GPU code (set-associative cache with device-side
  modify, GPU histogram, Deduper, gradient de-duplication, find_and_combine) compiled by nvcc for
  sm_100a from the reference checkout, wrapped by ``oracle/ref_gpu_driver.cu``.  Same rule: built
  only where the checkout is present.

* ``libnve_ref_ser.so`` – the UNMODIFIED reference weight-file code (``src/serialization.cpp``: the
  .nve container, the numpy and raw-binary table loaders), wrapped by
  ``oracle/ref_serialization_driver.cpp``.  Same rule.

No reference source is copied: the compiler reads the files where they lie.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
# the reference checkout: NVE_REFERENCE_DIR, else a directory named "reference" beside this repository
REFERENCE = Path(os.environ.get("NVE_REFERENCE_DIR", str(HERE.parents[1] / "reference")))

REF_SOURCES = [
    "host_embedding_layer", "linear_host_table", "host_table", "host_table_detail", "table",
    "layer_utils", "execution_context", "default_allocator", "thread_pool", "thread_pool_base",
    "common", "numa_support", "insert_heuristic",
]

REF_DEFINES = [
    "-DNVE_CACHE_LINE_SIZE=64", "-DNVE_DRIVERLESS_BUILD", "-DNVE_DISABLE_MPI",
    "-DNVE_FEATURE_HT_KEY_64=1", "-DNVE_FEATURE_HT_KEY_32=1", "-DNVE_FEATURE_HT_PART_FNV1A=1",
    "-DNVE_FEATURE_HT_KERNEL_8=1",
]


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def _find_nlohmann() -> Path | None:
    site = Path(sysconfig.get_paths()["purelib"])
    cand = site / "include" / "cudnn_frontend" / "thirdparty"
    if (cand / "nlohmann" / "json.hpp").exists():
        return cand
    for p in site.rglob("nlohmann/json.hpp"):
        return p.parent.parent
    return None


def build_oracle(verbose: bool = False) -> Path:
    """Compile the C restatement with gcc.  -ffp-contract=off keeps a*b+c unfused so that the
    arithmetic is the same on every host the library is rebuilt on."""
    OUT.mkdir(exist_ok=True)
    srcs = [HERE / "nve_oracle.c", HERE / "nve_oracle_cache.c"]
    out = OUT / "libnve_oracle.so"
    if _newer(out, srcs):
        return out
    cmd = ["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
           "-Wall", "-Wextra", "-o", str(out), *map(str, srcs), "-lm"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


AVX512_FLAGS = ["-mavx512f", "-mavx512bw", "-mavx512vl", "-mavx512vbmi"]


def host_has_avx512() -> bool:
    """Whether this host has the AVX-512 subsets the reference's build asks for when it finds them
    (cmake/nve_avx.cmake: F, BW, VL, VBMI)."""
    try:
        flags = set()
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                flags = set(line.split(":", 1)[1].split())
                break
        return {"avx512f", "avx512bw", "avx512vl", "avx512vbmi"} <= flags
    except OSError:
        return False


def build_reference(verbose: bool = False, avx512: bool = False) -> Path | None:
    """Compile the reference CPU path from its own sources (only where the checkout exists).
    The -mavx2 build is the one the parity pins use (no fused multiply-add on any host); the
    AVX-512 build (the flags the reference's cmake picks on a host that has them) exists for timing
    the CPU baseline on such hosts."""
    OUT.mkdir(exist_ok=True)
    out = OUT / ("libnve_ref_avx512.so" if avx512 else "libnve_ref.so")
    if not (REFERENCE / "src" / "host_embedding_layer.cpp").exists():
        return out if out.exists() else None
    driver = HERE / "ref_driver.cpp"
    if _newer(out, [driver]):
        return out
    nl = _find_nlohmann()
    if nl is None:
        raise RuntimeError("nlohmann/json.hpp not found in site-packages")
    shim = OUT / "shim" / "nlohmann"
    shim.mkdir(parents=True, exist_ok=True)
    (shim / "json_fwd.hpp").write_text("#pragma once\n#include <nlohmann/json.hpp>\n")
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    cmd = ["g++", "-std=c++17", "-O3", *(AVX512_FLAGS if avx512 else ["-mavx2"]), "-fPIC", "-shared", "-w",
           *REF_DEFINES,
           f"-I{REFERENCE}", f"-I{REFERENCE / 'include'}", f"-I{cuda_inc}", f"-I{nl}",
           f"-I{shim.parent}", str(driver),
           *[str(REFERENCE / "src" / f"{s}.cpp") for s in REF_SOURCES],
           "-o", str(out),
           f"-L{cuda_inc.parent / 'lib64'}", "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


def _shim_and_json():
    nl = _find_nlohmann()
    if nl is None:
        raise RuntimeError("nlohmann/json.hpp not found in site-packages")
    shim = OUT / "shim" / "nlohmann"
    shim.mkdir(parents=True, exist_ok=True)
    (shim / "json_fwd.hpp").write_text("#pragma once\n#include <nlohmann/json.hpp>\n")
    return nl, shim.parent


def build_reference_gpu(verbose: bool = False) -> Path | None:
    """Compile the reference GPU code (header templates + two support sources) with nvcc for
    sm_100a, with the reference's own fast-math setting and NDEBUG as in its release build (its
    size self-check asserts otherwise abort on a cache sized to a whole number of sets).  About
    half a minute."""
    OUT.mkdir(exist_ok=True)
    out = OUT / "libnve_ref_gpu.so"
    if not (REFERENCE / "cuda_ops" / "deduper.cuh").exists():
        return out if out.exists() else None
    driver = HERE / "ref_gpu_driver.cu"
    if _newer(out, [driver]):
        return out
    nl, shim = _shim_and_json()
    nvcc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    cmd = [str(nvcc), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
           "--expt-relaxed-constexpr", "--use_fast_math", "-w", "-Xcompiler", "-fPIC", "-shared",
           "-cudart", "static", "-DNDEBUG", "-DNVE_CACHE_LINE_SIZE=64", "-DNVE_DISABLE_MPI",
           f"-I{REFERENCE}", f"-I{REFERENCE / 'include'}", f"-I{REFERENCE / 'include' / 'ecache'}",
           f"-I{nl}", f"-I{shim}", str(driver),
           str(REFERENCE / "src" / "default_allocator.cpp"), str(REFERENCE / "src" / "common.cpp"),
           "-o", str(out)]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


def build_reference_serialization(verbose: bool = False) -> Path | None:
    """Compile the reference weight-file code (src/serialization.cpp) with g++ behind
    ``oracle/ref_serialization_driver.cpp`` (only where the checkout exists)."""
    OUT.mkdir(exist_ok=True)
    out = OUT / "libnve_ref_ser.so"
    if not (REFERENCE / "src" / "serialization.cpp").exists():
        return out if out.exists() else None
    driver = HERE / "ref_serialization_driver.cpp"
    if _newer(out, [driver]):
        return out
    nl, shim = _shim_and_json()
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w", *REF_DEFINES,
           f"-I{REFERENCE}", f"-I{REFERENCE / 'include'}", f"-I{cuda_inc}", f"-I{nl}", f"-I{shim}",
           str(driver), str(REFERENCE / "src" / "serialization.cpp"), str(REFERENCE / "src" / "common.cpp"),
           "-o", str(out)]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


def build_all(verbose: bool = False):
    build_reference(verbose, avx512=True)
    return (build_oracle(verbose), build_reference(verbose), build_reference_gpu(verbose),
            build_reference_serialization(verbose))


if __name__ == "__main__":
    o, r, g, w = build_all(verbose=True)
    print("oracle:", o)
    print("reference:", r)
    print("reference (GPU):", g)
    print("reference (weight files):", w)
    sys.exit(0)
