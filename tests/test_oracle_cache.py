"""Known-answer tests of the C restatement of the set-associative cache.  The scenarios restate
the reference's own ecache API tests (tests/ecache/api_test.cu) and replacement scenarios
(tests/kernels/gpu_insert_tests.cu) as procedures on seeded data."""
import numpy as np
import pytest

from oracle.pyoracle import OracleCache

ROW = 64


def per_set(row=ROW, key_bytes=8):
    return 8 * key_bytes + 8 * row + 32


def table(rows, row=ROW, seed=0):
    """Row r holds r in its first 8 bytes, then a seeded pattern."""
    t = np.random.default_rng(seed).integers(0, 256, (rows, row), dtype=np.uint8)
    t[:, :8] = np.arange(rows, dtype=np.int64).view(np.uint8).reshape(rows, 8)
    return t


@pytest.mark.parametrize("key_dtype", [np.int32, np.int64])
def test_geometry(oracle, key_dtype):
    kb = np.dtype(key_dtype).itemsize
    c = OracleCache(oracle, 100 * per_set(ROW, kb) + 17, ROW, key_dtype)
    assert c.num_sets == 100
    # the large-cache arithmetic: 2.56e9 bytes of 256-byte rows with int64 tags
    assert oracle.lib.nve_oracle_cache_num_sets(2_560_000_000, 256, 8) == 2_560_000_000 // 2144 == 1_194_029


@pytest.mark.parametrize("key_dtype", [np.int32, np.int64])
def test_empty_cache_reports_every_key_missing_in_order(oracle, key_dtype):
    c = OracleCache(oracle, 16 * per_set(), ROW, key_dtype)
    keys = np.array([5, 9, 1, 1000, 7], dtype=key_dtype)
    out = np.full((5, ROW), 0xEE, dtype=np.uint8)
    n, pos, mk = c.lookup(keys, out, want_miss_list=True)
    assert n == 5 and pos.tolist() == [0, 1, 2, 3, 4] and mk.tolist() == keys.tolist()
    assert c.misses == 5
    assert (out == 0xEE).all()
    assert c.resident_keys().size == 0


@pytest.mark.parametrize("key_dtype", [np.int32, np.int64])
def test_insert_lookup_invalidate_clear(oracle, key_dtype):
    t = table(1000)
    c = OracleCache(oracle, 16 * per_set(), ROW, key_dtype)
    keys = np.arange(10, dtype=key_dtype)
    assert c.insert(keys, values=t[:10]) == 10
    assert sorted(c.resident_keys().tolist()) == list(range(10))
    out = np.zeros((10, ROW), dtype=np.uint8)
    c.reset_misses()
    assert c.lookup(keys, out) == 0 and c.misses == 0
    assert np.array_equal(out, t[:10])
    # hit mask: bit i set for resolved keys; pre-set bits are skipped
    mask = np.array([0b100], dtype=np.uint64)
    out2 = np.zeros((12, ROW), dtype=np.uint8)
    probe = np.array(list(range(10)) + [500, 501], dtype=key_dtype)
    assert c.lookup(probe, out2, hit_mask=mask) == 2
    assert int(mask[0]) == 0b1111111111
    assert not out2[2].any() and np.array_equal(out2[3], t[3])
    # backed lookup resolves the rest from the table and still counts them as cache misses
    c.reset_misses()
    out3 = np.zeros((12, ROW), dtype=np.uint8)
    assert c.lookup(probe, out3, table=t) == 0 and c.misses == 2
    assert np.array_equal(out3, t[probe])
    # invalidate {3, 7}: exactly those leave, and miss in that order
    c.invalidate(np.array([3, 7], dtype=key_dtype))
    assert sorted(c.resident_keys().tolist()) == [0, 1, 2, 4, 5, 6, 8, 9]
    n, pos, mk = c.lookup(keys, out, want_miss_list=True)
    assert (n, pos.tolist(), mk.tolist()) == (2, [3, 7], [3, 7])
    c.clear()
    assert c.resident_keys().size == 0


def test_negative_keys_round_trip(oracle):
    """Negative keys other than the sentinel are ordinary keys (unsigned hashing)."""
    c = OracleCache(oracle, 13 * per_set(), ROW, np.int64)
    keys = np.array([-2, -3, -100, -(1 << 40), 5], dtype=np.int64)
    vals = table(5, seed=3)
    assert c.insert(keys, values=vals) == 5
    assert sorted(c.resident_keys().tolist()) == sorted(keys.tolist())
    out = np.zeros((5, ROW), dtype=np.uint8)
    assert c.lookup(keys, out) == 0
    assert np.array_equal(out, vals)
    c32 = OracleCache(oracle, 13 * per_set(ROW, 4), ROW, np.int32)
    k32 = np.array([-2, -3, -100, 5], dtype=np.int32)
    assert c32.insert(k32, values=vals[:4]) == 4
    assert sorted(c32.resident_keys().tolist()) == sorted(k32.tolist())


def test_update_and_update_accumulate(oracle):
    rows = 64
    t = np.random.default_rng(1).normal(size=(rows, 16)).astype(np.float32)
    tb = t.view(np.uint8).reshape(rows, 64)
    c = OracleCache(oracle, 8 * per_set(), ROW, np.int64)
    c.insert(np.arange(20, dtype=np.int64), values=tb[:20])
    upd = np.zeros((3, 16), dtype=np.float32)
    upd[:, 0] = 1.0
    c.update_accumulate(np.array([2, 5, 63], dtype=np.int64), upd)   # 63 is not resident
    out = np.zeros((20, 64), dtype=np.uint8)
    c.lookup(np.arange(20, dtype=np.int64), out)
    got = out.view(np.float32)
    want = t[:20].copy()
    want[[2, 5], 0] += 1.0
    assert np.array_equal(got, want)       # exact fp32 equality, as the reference test demands
    new_rows = np.full((2, 64), 7, dtype=np.uint8)
    c.update(np.array([0, 40], dtype=np.int64), new_rows)
    c.lookup(np.arange(20, dtype=np.int64), out)
    assert (out[0] == 7).all() and np.array_equal(out[1:].view(np.float32), want[1:])
    assert 40 not in c.resident_keys().tolist()


def test_low_priority_never_evicts_high_priority_does(oracle):
    sets = 8
    c = OracleCache(oracle, sets * per_set(), ROW, np.int64, decay_rate=0.95)
    lines = sets * 8
    t = table(10_000)
    resident = np.arange(lines, dtype=np.int64)
    assert c.insert(np.repeat(resident, 4), table=t) == lines          # every line, priority 1/lines
    before = c.tags().copy()
    foreign = (np.arange(8, dtype=np.int64) + 100) * sets              # 8 new keys, all in set 0
    filler = np.tile(resident[resident % sets != 0], 3)                # hits only: they lower 1/n
    assert c.insert(np.concatenate([foreign, filler]), table=t) == 0   # 1/n < 0.95/lines: no change
    assert np.array_equal(c.tags(), before)
    assert c.insert(np.repeat(foreign, 100), table=t) == 8             # priority 1/8 beats everything
    assert sorted(c.resident_keys()[:8].tolist()) == sorted(foreign.tolist())
    out = np.zeros((8, ROW), dtype=np.uint8)
    assert c.lookup(foreign, out) == 0 and np.array_equal(out, t[foreign])


def test_replacement_counts_against_decayed_counters(oracle):
    """Counters 10/n decayed once to 9.5/n; new keys with counts 6..13 per set: exactly the four
    with counts 10..13 get in, replacing four ways; the rest of the set keeps its keys."""
    sets = 6                     # sets 0..4 under test, set 5 only carries padding keys
    c = OracleCache(oracle, sets * per_set(), ROW, np.int64, decay_rate=0.95)
    t = table(100_000)
    first = np.array([s + sets * w for s in range(5) for w in range(8)], dtype=np.int64)
    pad = np.array([5 + sets * w for w in range(8)], dtype=np.int64)
    n = 5 * 8 * 10 + 80
    batch1 = np.concatenate([np.repeat(first, 10), np.repeat(pad, 10)])
    assert batch1.size == n
    assert c.insert(batch1, table=t) == 48
    new = np.array([s + sets * (100 + w) for s in range(5) for w in range(8)], dtype=np.int64)
    counts = np.tile(np.arange(6, 14), 5)
    batch2 = np.concatenate([np.repeat(new, counts), np.repeat(pad[:1] + sets * 50, n - counts.sum())])
    assert batch2.size == n
    replaced = c.insert(batch2, table=t)
    assert replaced == 5 * 4 + 1     # four per tested set, plus the padding key in set 5
    res = set(c.resident_keys().tolist())
    for s in range(5):
        got_new = sorted(k for k in res if k % sets == s and k >= sets * 100)
        assert got_new == [s + sets * (100 + w) for w in (4, 5, 6, 7)]
        assert len([k for k in res if k % sets == s]) == 8


def test_more_than_eight_equal_candidates_per_set(oracle):
    """The selection network has no tie guard in its merge step: with more than 8 equal-priority
    new keys in one set, one key fills all 8 ways.  Kept (it is what decides residency)."""
    sets = 4
    c = OracleCache(oracle, sets * per_set(), ROW, np.int64)
    t = table(1000)
    keys = np.arange(20, dtype=np.int64) * sets          # 20 keys in set 0, each once
    assert c.insert(keys, table=t) == 8
    assert c.resident_keys().tolist() == [28] * 8        # the 8th key of the first chunk
    out = np.zeros((1, ROW), dtype=np.uint8)
    assert c.lookup(np.array([28], dtype=np.int64), out) == 0 and np.array_equal(out[0], t[28])


def test_max_modify_keeps_the_most_frequent(oracle):
    c = OracleCache(oracle, 64 * per_set(), ROW, np.int64)
    t = table(1000)
    keys = np.concatenate([np.arange(100), np.arange(10), np.arange(5)]).astype(np.int64)
    assert c.insert(keys, table=t, max_modify=10) == 10
    assert sorted(c.resident_keys().tolist()) == list(range(10))


def test_lazy_decay_uses_elapsed_inserts(oracle):
    sets = 4
    c = OracleCache(oracle, sets * per_set(), ROW, np.int64, decay_rate=0.5)
    t = table(1000)
    c.insert(np.array([0], dtype=np.int64), table=t)              # set 0: counter 1.0 at ts 1
    for k in (1, 5, 9):                                            # three inserts touching set 1 only
        c.insert(np.array([k], dtype=np.int64), table=t)
    assert c.counters()[0, :].max() == 1.0                         # untouched set not yet decayed
    c.insert(np.array([0], dtype=np.int64), table=t)              # hit: 1.0 * 0.5^4 + 1.0
    assert c.counters()[0].max() == np.float32(1.0 * 0.5 ** 4 + 1.0)
