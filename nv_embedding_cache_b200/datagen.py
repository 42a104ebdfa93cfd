"""Seeded synthetic workloads with the shapes and distributions of the benchmark configurations.

Everything here is numpy on the host and fully determined by its seeds, so the GPU box and a CPU
box produce identical bytes.  Key streams take the form of the reference's own generator
(samples/pytorch/pytorch_samples_common.py:21-46): a power law over row ranks mapped through a
seeded permutation of row ids.
"""
from __future__ import annotations

import numpy as np

PERM_SEED = 31337


def permutation(num_rows: int, seed: int = PERM_SEED) -> np.ndarray:
    return np.random.default_rng(seed).permutation(num_rows).astype(np.int64)


def power_law_ranks(n: int, num_rows: int, alpha: float, seed: int) -> np.ndarray:
    """rank = floor((x * (N^(1-a) - 1) + 1)^(1/(1-a))) for x ~ U[0,1), clamped to N-1."""
    x = np.random.default_rng(seed).random(n)
    e = 1.0 - alpha
    y = (x * (float(num_rows) ** e - 1.0) + 1.0) ** (1.0 / e)
    r = y.astype(np.int64)
    np.minimum(r, num_rows - 1, out=r)
    return r


def affine_permute(ranks: np.ndarray, num_rows: int, seed: int = PERM_SEED) -> np.ndarray:
    """Permutation of [0, num_rows) without a table: r -> (a*r + b) mod N with gcd(a, N) = 1.
    Used where an explicit permutation array would not fit comfortably in host memory."""
    rng = np.random.default_rng(seed)
    a = int(rng.integers(num_rows // 3, num_rows)) | 1
    while np.gcd(a, num_rows) != 1:
        a += 2
    b = int(rng.integers(0, num_rows))
    # 128-bit safe: split multiplication through Python ints only when it could overflow
    if num_rows < (1 << 31):
        return ((ranks.astype(np.uint64) * np.uint64(a) + np.uint64(b)) % np.uint64(num_rows)).astype(np.int64)
    out = np.empty_like(ranks)
    for i, r in enumerate(ranks.tolist()):
        out[i] = (a * r + b) % num_rows
    return out


def zipf_keys(n: int, num_rows: int, alpha: float, seed: int, perm: np.ndarray | None = None) -> np.ndarray:
    ranks = power_law_ranks(n, num_rows, alpha, seed)
    if perm is not None:
        return perm[ranks]
    return affine_permute(ranks, num_rows)


def uniform_keys(n: int, num_rows: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, num_rows, n, dtype=np.int64)


def csr_bags(num_bags: int, lo: int, hi: int, seed: int):
    """Bag lengths uniform in [lo, hi]; returns (lengths, offsets with trailing total)."""
    lengths = np.random.default_rng(seed).integers(lo, hi + 1, num_bags, dtype=np.int64)
    offsets = np.zeros(num_bags + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    return lengths, offsets


def dyadic_table(num_rows: int, width: int, seed: int, dtype=np.float32) -> np.ndarray:
    """Values a / 2^b with a in [-8, 8], b in [3, 9]: sums of a few hundred such values are exact
    in fp32 (and, for short bags, in fp16), so an unweighted Sum has one right answer whatever the
    order."""
    rng = np.random.default_rng(seed)
    a = rng.integers(-8, 9, (num_rows, width)).astype(np.float32)
    b = rng.integers(3, 10, (num_rows, width)).astype(np.float32)
    return (a / np.exp2(b)).astype(dtype)


def normal_table(num_rows: int, width: int, std: float, seed: int, dtype=np.float16) -> np.ndarray:
    rng = np.random.default_rng(seed)
    out = np.empty((num_rows, width), dtype=dtype)
    step = max(1, (1 << 22) // max(1, width))
    for r0 in range(0, num_rows, step):
        r1 = min(num_rows, r0 + step)
        out[r0:r1] = rng.standard_normal((r1 - r0, width), dtype=np.float32) * std
    return out


def quantized_rows(num_rows: int, width: int, seed: int, value_dtype: str = "qint8_f32",
                   stride: int | None = None) -> np.ndarray:
    """Row-wise quantised rows: `width` int8/uint8 values, then scale (and offset for uint8) in
    fp32 or fp16 directly after the values, then padding up to `stride` bytes.  Scale is uniform in
    [1e-3, 1e-2]; offsets uniform in [-0.5, 0.5]."""
    signed = value_dtype.startswith("qint8")
    meta_t = np.float32 if value_dtype.endswith("f32") else np.float16
    n_meta = 1 if signed else 2
    meta_bytes = n_meta * np.dtype(meta_t).itemsize
    tight = width + meta_bytes
    stride = tight if stride is None else stride
    assert stride >= tight
    rng = np.random.default_rng(seed)
    rows = np.zeros((num_rows, stride), dtype=np.uint8)
    if signed:
        rows[:, :width] = rng.integers(-127, 128, (num_rows, width)).astype(np.int8).view(np.uint8)
    else:
        rows[:, :width] = rng.integers(0, 256, (num_rows, width)).astype(np.uint8)
    meta = np.empty((num_rows, n_meta), dtype=meta_t)
    meta[:, 0] = rng.uniform(1e-3, 1e-2, num_rows).astype(meta_t)
    if not signed:
        meta[:, 1] = rng.uniform(-0.5, 0.5, num_rows).astype(meta_t)
    rows[:, width:tight] = meta.view(np.uint8).reshape(num_rows, meta_bytes)
    return rows
