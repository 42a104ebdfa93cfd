"""Pins the C restatement (oracle/nve_oracle.c): bit-for-bit against the committed golden vectors
(outputs of the unmodified reference CPU path) and, where the reference build is available,
against that build run live on further seeded cases."""
import numpy as np
import pytest

from golden.cases import build_cases
from nv_embedding_cache_b200 import datagen as dg
from pathlib import Path

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_outputs.npz")
CASES = build_cases()


def run_oracle(oracle, case):
    table = case["table"].copy()
    if case["op"] == "gather":
        out = np.zeros((case["keys"].size, table.shape[1]), dtype=np.uint8)
        assert oracle.gather(table, case["keys"], out) == case["keys"].size
        return out
    if case["op"] == "accumulate":
        t = table.view(np.float32)
        oracle.update_accumulate(t, case["keys"], case["updates"])
        return t
    return oracle.lookup_pooled(table, case["value_dtype"], case["width"], case["keys"],
                                case["pooling"], offsets=case["offsets"], hotness=case["hotness"],
                                weights=case["weights"], out_dtype=case["out_dtype"])


def test_golden_file_covers_every_case():
    assert set(GOLDEN.files) == set(CASES)


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_golden_bit_for_bit(oracle, name):
    got = run_oracle(oracle, CASES[name])
    want = GOLDEN[name]
    assert got.shape == want.shape and got.dtype == want.dtype
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_dyadic_sums_are_exact(oracle):
    """On dyadic tables the fp32 sum has one right answer: compare with float64 arithmetic."""
    case = CASES["f32_w132_fixed59_sum_dyadic"]
    t = case["table"].view(np.float32)
    want = t[case["keys"]].astype(np.float64).reshape(17, 59, 132).sum(1)
    assert np.array_equal(GOLDEN["f32_w132_fixed59_sum_dyadic"].astype(np.float64), want)


@pytest.mark.parametrize("seed", range(6))
def test_oracle_matches_live_reference(oracle, reference, seed):
    rng = np.random.default_rng(1000 + seed)
    vd = ["f32", "f16", "qint8_f32", "qint8_f16", "quint8_f32", "quint8_f16"][seed]
    width = int(rng.choice([2, 30, 63, 64, 128, 132, 256]))
    rows = 777
    if vd == "f32":
        table = dg.normal_table(rows, width, 0.5, seed, np.float32).view(np.uint8).reshape(rows, -1)
    elif vd == "f16":
        table = dg.normal_table(rows, width, 0.5, seed, np.float16).view(np.uint8).reshape(rows, -1)
    else:
        table = dg.quantized_rows(rows, width, seed, vd)
    layer = reference.layer(table, vd)
    for pooling in ("sum", "mean", "wsum", "wmean"):
        for out_dtype in ("f32", "f16"):
            _, offs = dg.csr_bags(33, 0, 40, seed * 7 + 1)
            keys = dg.uniform_keys(int(offs[-1]), rows, seed + 50)
            w = rng.uniform(-1, 1, keys.size).astype(np.float32) if pooling.startswith("w") else None
            a = oracle.lookup_pooled(table, vd, width, keys, pooling, offsets=offs, weights=w,
                                     out_dtype=out_dtype)
            b = layer.lookup_pooled(keys, pooling, width, offsets=offs, weights=w, out_dtype=out_dtype)
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), (vd, width, pooling, out_dtype)
    layer.close()


def test_int32_offsets_match_reference(oracle, reference):
    case = CASES["f16_w128_csr_mean"]
    offs32 = case["offsets"].astype(np.int32)
    gathered = case["table"][case["keys"]]
    layer = reference.layer(case["table"], "f16")
    want = layer.pool_gathered_i32(gathered, 128, "mean", offs32, out_dtype="f16")
    got = oracle.lookup_pooled(case["table"], "f16", 128, case["keys"], "mean", offsets=offs32,
                               out_dtype="f16")
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    assert np.array_equal(got.view(np.uint16), GOLDEN["f16_w128_csr_mean"].view(np.uint16))
    layer.close()


def test_gather_skips_out_of_range_and_honours_hit_mask(oracle):
    t = np.arange(40, dtype=np.float32).reshape(10, 4)
    keys = np.array([3, -1, 10, 0, 9, 5], dtype=np.int64)
    out = np.full((6, 4), -7, dtype=np.float32)
    mask = np.array([1 << 5], dtype=np.uint64)  # key 5 already resolved
    hits = oracle.gather(t, keys, out, mask)
    assert hits == 3
    assert int(mask[0]) == 0b111001
    assert np.array_equal(out[0], t[3]) and np.array_equal(out[3], t[0]) and np.array_equal(out[4], t[9])
    assert (out[1] == -7).all() and (out[2] == -7).all() and (out[5] == -7).all()


def test_c1_configuration_at_full_size_matches_live_reference(oracle, reference):
    """The reference's CPU-runnable configuration with its own inputs and sizes: 1 000 000 x 64 fp32
    uniform[-0.05, 0.05] (seed 1), 8192 bags x 16 Zipf(1.05) keys over a permuted row order, fp32
    sums -- the oracle against the reference's HostEmbeddingLayer, every bit of all 8192 x 64 sums.
    (The GPU test of the same configuration compares the library with the oracle.)"""
    rows, dim, bags, hot = 1_000_000, 64, 8192, 16
    table = np.random.default_rng(1).uniform(-0.05, 0.05, (rows, dim)).astype(np.float32)
    keys = dg.zipf_keys(bags * hot, rows, 1.05, 1000, dg.permutation(rows))
    tb = table.view(np.uint8).reshape(rows, -1)
    a = oracle.lookup_pooled(tb, "f32", dim, keys, "sum", hotness=hot, out_dtype="f32")
    layer = reference.layer(tb, "f32")
    b = layer.lookup_pooled(keys, "sum", dim, hotness=hot, out_dtype="f32")
    layer.close()
    assert a.shape == (bags, dim)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
