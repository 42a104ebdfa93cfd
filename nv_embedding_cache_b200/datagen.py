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
    # a, r < 2^32 keeps a * r inside 64 bits; larger tables go through Python integers
    if num_rows < (1 << 32):
        n = np.uint64(num_rows)
        return (((ranks.astype(np.uint64) * np.uint64(a)) % n + np.uint64(b)) % n).astype(np.int64)
    out = np.empty_like(ranks)
    for i, r in enumerate(ranks.tolist()):
        out[i] = (a * r + b) % num_rows
    return out


def zipf_keys(n: int, num_rows: int, alpha: float, seed: int, perm: np.ndarray | None = None) -> np.ndarray:
    ranks = power_law_ranks(n, num_rows, alpha, seed)
    if perm is not None:
        return perm[ranks]
    return affine_permute(ranks, num_rows)


_MASK64 = (1 << 64) - 1


def hashed_rows_f16(row_ids: np.ndarray, width: int, seed: int, scale: float = 0.08) -> np.ndarray:
    """Rows of a table too large to generate with a sequential generator: element (r, c) is a
    function of (seed, r, c) alone -- an 11-bit field of a splitmix64 hash, centred and scaled to
    [-scale/2, scale/2) -- so any subset of rows can be produced anywhere.  The device-side twin is
    fill_hashed_rows_f16 (torch); both give the same bytes."""
    r = np.asarray(row_ids, dtype=np.uint64).reshape(-1, 1)
    c = np.arange(width, dtype=np.uint64).reshape(1, -1)
    with np.errstate(over="ignore"):
        x = r * np.uint64(width) + c + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        x = x ^ (x >> np.uint64(31))
    f = (x >> np.uint64(53)).astype(np.float32) * np.float32(2.0 ** -11) - np.float32(0.5)
    return (f * np.float32(scale)).astype(np.float16)


def fill_hashed_rows_f16(dst, first_row: int, row_step: int, seed: int, scale: float = 0.08,
                         chunk_rows: int = 1 << 21):
    """dst[i] = hashed_rows_f16([first_row + i * row_step]) for a torch fp16 tensor [rows, width] on
    any device, computed chunk-wise on dst's device with 64-bit integer tensor arithmetic (which
    wraps like the numpy form; logical shifts are arithmetic shifts with the sign bits masked)."""
    import torch
    rows, width = dst.shape
    dev = dst.device if dst.device.type == "cuda" else torch.device("cuda", torch.cuda.current_device())

    def wrap(v):      # Python int -> the int64 with the same low 64 bits
        v &= _MASK64
        return v - (1 << 64) if v >= (1 << 63) else v

    def shr(x, k):
        return (x >> k) & ((1 << (64 - k)) - 1)
    c = torch.arange(width, dtype=torch.int64, device=dev).reshape(1, -1)
    salt = wrap(seed * 0x9E3779B97F4A7C15)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        r = (torch.arange(r0, r1, dtype=torch.int64, device=dev) * row_step + first_row).reshape(-1, 1)
        x = r * width + c + salt
        x = (x ^ shr(x, 30)) * wrap(0xBF58476D1CE4E5B9)
        x = (x ^ shr(x, 27)) * wrap(0x94D049BB133111EB)
        x = x ^ shr(x, 31)
        f = shr(x, 53).to(torch.float32) * (2.0 ** -11) - 0.5
        dst[r0:r1].copy_((f * scale).to(torch.float16))


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
