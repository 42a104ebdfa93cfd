"""Known-answer tests of the Deduper restatement (procedures of the reference's
tests/kernels/deduper_tests.cu:118-348)."""
import numpy as np

from nv_embedding_cache_b200 import datagen as dg


def check_contract(keys, d):
    """unique/counts/offsets/inverse describe the batch exactly once."""
    u = d["unique"]
    assert np.all(np.diff(u) > 0)
    assert d["counts"].sum() == keys.size
    starts = np.concatenate([[0], np.cumsum(d["counts"])])
    seen = np.zeros(keys.size, dtype=bool)
    for i in range(d["num_unique"]):
        pos = d["inverse"][starts[i]:starts[i + 1]]
        assert np.all(keys[pos] == u[i]) and np.all(np.diff(pos) > 0)
        seen[pos] = True
    assert seen.all()


def test_all_unique_all_identical_empty_single(oracle):
    k = np.array([9, 3, 7, 1], dtype=np.int64)
    d = oracle.dedup(k)
    assert d["unique"].tolist() == [1, 3, 7, 9] and d["counts"].tolist() == [1, 1, 1, 1]
    assert d["inverse"].tolist() == [3, 1, 2, 0] and d["offsets"].tolist() == [0, 1, 2, 3, 4]
    d = oracle.dedup(np.full(6, 42, dtype=np.int64))
    assert (d["num_unique"], d["unique"].tolist(), d["counts"].tolist()) == (1, [42], [6])
    assert d["inverse"].tolist() == list(range(6))
    d = oracle.dedup(np.zeros(0, dtype=np.int64))
    assert d["num_unique"] == 0 and d["num_chunks"] == 0
    d = oracle.dedup(np.array([5], dtype=np.int64))
    assert d["unique"].tolist() == [5] and d["offsets"].tolist() == [0, 1]


def test_split_long_run(oracle):
    """20 copies of one key + 5 singles, max run 8: 6 unique keys, chunks 8, 8, 4, then 1 x 5."""
    k = np.array([100] * 20 + [1, 2, 3, 4, 5], dtype=np.int64)
    d = oracle.dedup(k, max_run=8)
    assert d["num_unique"] == 6 and d["num_chunks"] == 8
    assert d["unique"].tolist() == [1, 2, 3, 4, 5, 100]
    assert np.diff(d["offsets"]).tolist() == [1, 1, 1, 1, 1, 8, 8, 4]
    assert d["loc_map"].tolist() == [0, 1, 2, 3, 4, 5, 5, 5]
    check_contract(k, d)


def test_reduced_end_bit_and_random_round_trip(oracle):
    k = np.array([0x105, 0x005, 0x203, 0x003], dtype=np.int64)
    d = oracle.dedup(k, end_bit=8)   # only the low byte orders the keys; runs compare full keys
    assert d["unique"].tolist() == [0x203, 0x003, 0x105, 0x005] and d["counts"].tolist() == [1, 1, 1, 1]
    assert d["inverse"].tolist() == [2, 3, 0, 1]
    k = np.array([200, 7, 200, 3, 7, 255], dtype=np.int64)
    d = oracle.dedup(k, end_bit=8)   # keys below 2^end_bit: identical to the full sort
    full = oracle.dedup(k)
    assert all(np.array_equal(d[x], full[x]) for x in ("unique", "counts", "inverse", "offsets"))
    keys = dg.zipf_keys(5000, 800, 1.05, 3, dg.permutation(800))
    d = oracle.dedup(keys, max_run=16)
    check_contract(keys, d)
    assert np.array_equal(d["unique"], np.unique(keys))
    neg = np.array([-5, 3, -5, -1, 3, 0], dtype=np.int64)
    d = oracle.dedup(neg)
    assert d["unique"].tolist() == [-5, -1, 0, 3]


def test_grad_sums(oracle):
    keys = dg.zipf_keys(3000, 200, 1.1, 4, dg.permutation(200))
    grads = dg.dyadic_table(3000, 12, 5, np.float32)
    for max_run in (-1, 16):
        d = oracle.dedup(keys, max_run=max_run)
        got = oracle.dedup_grads(grads, d)
        want = np.zeros((d["num_unique"], 12), np.float64)
        np.add.at(want, np.searchsorted(d["unique"], keys), grads.astype(np.float64))
        assert np.array_equal(got.astype(np.float64), want)   # dyadic values: exact in any order
