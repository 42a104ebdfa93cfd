"""Seeded small cases shared by the golden-vector generator and the parity tests.

Each case builds its inputs from numpy seeds only; the expected outputs stored in
``reference_outputs.npz`` were produced by the unmodified reference CPU path
(``make_golden.py``).  Shapes follow the reference's own kernel tests: widths that force 16-, 4-
and element-sized vectors (132, 30, 63), hotness 59, batch 17, dyadic tables for exact sums,
weights of 0.5 / 0.25, empty bags.
"""
from __future__ import annotations

import numpy as np

from nv_embedding_cache_b200 import datagen as dg


def _bytes(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint8).reshape(a.shape[0], -1)


def _weights(n, seed, dtype=np.float32):
    return np.where(np.random.default_rng(seed).integers(0, 2, n) == 0, 0.5, 0.25).astype(dtype)


def build_cases():
    cases = {}

    def add(name, **kw):
        kw.setdefault("offsets", None)
        kw.setdefault("hotness", 0)
        kw.setdefault("weights", None)
        kw.setdefault("out_dtype", "f32")
        kw.setdefault("op", "pooled")
        cases[name] = kw

    # HostLayer-shaped sum: fp32 x 64, fixed hotness 16
    t = np.random.default_rng(1).uniform(-0.05, 0.05, (1000, 64)).astype(np.float32)
    add("f32_w64_fixed16_sum", table=_bytes(t), value_dtype="f32", width=64, pooling="sum",
        keys=dg.zipf_keys(64 * 16, 1000, 1.05, 101, dg.permutation(1000)), hotness=16)

    # GPULayer-shaped mean: fp16 x 128, CSR bags of 0..32 keys (empty bags included)
    t = dg.normal_table(5000, 128, 0.02, 20)
    _, offs = dg.csr_bags(300, 0, 32, 21)
    add("f16_w128_csr_mean", table=_bytes(t), value_dtype="f16", width=128, pooling="mean",
        keys=dg.zipf_keys(int(offs[-1]), 5000, 1.1, 102, dg.permutation(5000)), offsets=offs,
        out_dtype="f16")

    # dyadic tables, hotness 59, batch 17, widths 132 / 30 / 63
    for width, dt, npdt in ((132, "f32", np.float32), (30, "f16", np.float16),
                            (63, "f32", np.float32), (63, "f16", np.float16)):
        t = dg.dyadic_table(4096, width, 30 + width, npdt)
        add(f"{dt}_w{width}_fixed59_sum_dyadic", table=_bytes(t), value_dtype=dt, width=width,
            pooling="sum", keys=dg.zipf_keys(17 * 59, 4096, 1.05, 283982, dg.permutation(4096)),
            hotness=59, out_dtype=dt)

    # weighted CSR, bags of 1..31
    t = dg.dyadic_table(4096, 63, 40, np.float32)
    _, offs = dg.csr_bags(64, 1, 31, 0x475381)
    n = int(offs[-1])
    add("f32_w63_csr_wsum", table=_bytes(t), value_dtype="f32", width=63, pooling="wsum",
        keys=dg.zipf_keys(n, 4096, 1.05, 103, dg.permutation(4096)), offsets=offs,
        weights=_weights(n, 5))
    t = dg.normal_table(4096, 128, 0.02, 41)
    add("f16_w128_csr_wmean_w16", table=_bytes(t), value_dtype="f16", width=128, pooling="wmean",
        keys=dg.zipf_keys(n, 4096, 1.05, 104, dg.permutation(4096)), offsets=offs,
        weights=_weights(n, 6, np.float16), out_dtype="f16")

    # quantised rows: int8 + fp32 scale (tight 260-byte rows) -> fp16 sums
    q = dg.quantized_rows(2000, 256, 9, "qint8_f32")
    add("qint8f32_w256_fixed20_sum_f16", table=q, value_dtype="qint8_f32", width=256,
        pooling="sum", keys=dg.zipf_keys(50 * 20, 2000, 1.05, 105, dg.permutation(2000)),
        hotness=20, out_dtype="f16")
    q = dg.quantized_rows(2000, 252, 10, "qint8_f32")
    add("qint8f32_w252_fixed20_mean_f32", table=q, value_dtype="qint8_f32", width=252,
        pooling="mean", keys=dg.zipf_keys(50 * 20, 2000, 1.05, 106, dg.permutation(2000)),
        hotness=20)
    q = dg.quantized_rows(1500, 30, 11, "quint8_f16")
    _, offs = dg.csr_bags(40, 0, 17, 12)
    n = int(offs[-1])
    add("quint8f16_w30_csr_wmean_f32", table=q, value_dtype="quint8_f16", width=30,
        pooling="wmean", keys=dg.zipf_keys(n, 1500, 1.05, 107, dg.permutation(1500)),
        offsets=offs, weights=_weights(n, 7))
    q = dg.quantized_rows(1500, 64, 13, "quint8_f32")
    add("quint8f32_w64_fixed8_sum_f32", table=q, value_dtype="quint8_f32", width=64,
        pooling="sum", keys=dg.zipf_keys(32 * 8, 1500, 1.05, 108, dg.permutation(1500)), hotness=8)
    q = dg.quantized_rows(1500, 128, 14, "qint8_f16")
    add("qint8f16_w128_fixed4_mean_f16", table=q, value_dtype="qint8_f16", width=128,
        pooling="mean", keys=dg.zipf_keys(64 * 4, 1500, 1.05, 109, dg.permutation(1500)),
        hotness=4, out_dtype="f16")

    # Concatenate with dequantisation / conversion (one output row per key)
    add("qint8f16_w128_concat_f16", table=q, value_dtype="qint8_f16", width=128, pooling="concat",
        keys=dg.zipf_keys(200, 1500, 1.05, 110, dg.permutation(1500)), out_dtype="f16")
    t = dg.normal_table(3000, 96, 0.02, 42)
    add("f16_w96_concat_f32", table=_bytes(t), value_dtype="f16", width=96, pooling="concat",
        keys=dg.zipf_keys(333, 3000, 1.05, 111, dg.permutation(3000)), out_dtype="f32")

    # plain un-pooled lookup (raw rows)
    add("f16_w128_gather", table=_bytes(t[:, :96]).copy(), value_dtype="f16", width=96, op="gather",
        pooling="concat", keys=dg.zipf_keys(777, 3000, 1.2, 112, dg.permutation(3000)), out_dtype="f16")

    # update_accumulate on unique keys (SGD-style: -lr * grad)
    t = dg.normal_table(512, 64, 0.02, 43, np.float32)
    keys = np.random.default_rng(44).permutation(512)[:200].astype(np.int64)
    upd = (-0.01 * np.random.default_rng(45).normal(0, 1e-2, (200, 64))).astype(np.float32)
    add("f32_w64_update_accumulate", table=_bytes(t), value_dtype="f32", width=64, op="accumulate",
        pooling="concat", keys=keys, updates=upd)
    return cases
