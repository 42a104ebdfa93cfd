"""The host-side replacement policy of the cache table (csrc/host/host_policy.hpp, used when a table
is created with modify_on_gpu = 0), compiled by itself and driven without a GPU, against a
restatement in Python of the reference's algorithm (include/ecache/ec_set_associative_host_modify.h:
217-316 insert with lazy per-set decay, 134-176 invalidate, 489-511 the search behind update; the
host histogram of include/ecache/embed_cache.h:199-229).  On a GPU the same policy is compared with
the reference's own class (tests/test_gpu_reference_gpu.py)."""
import ctypes as C
import math
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "nv_embedding_cache_b200" / "csrc"
DECAY = np.float32(0.95)


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = tmp_path_factory.mktemp("host_policy") / "libhost_policy_shim.so"
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-I{CSRC}",
                           str(ROOT / "tests" / "host_policy_shim.cpp"), "-o", str(out)])
    lib = C.CDLL(str(out))
    lib.hp_create.restype = C.c_void_p
    lib.hp_create.argtypes = [C.c_uint32, C.c_int64]
    lib.hp_destroy.argtypes = [C.c_void_p]
    p = C.c_void_p
    lib.hp_histogram.restype = C.c_int64
    lib.hp_histogram.argtypes = [p, C.c_int64, p, p, p]
    lib.hp_insert.restype = C.c_int64
    lib.hp_insert.argtypes = [p, p, C.c_int64, C.c_float, C.c_int64, p, p, p]
    lib.hp_find_resident.restype = C.c_int64
    lib.hp_find_resident.argtypes = [p, p, C.c_int64, C.c_int64, p, p]
    lib.hp_invalidate.restype = C.c_int64
    lib.hp_invalidate.argtypes = [p, p, C.c_int64, p]
    lib.hp_state.argtypes = [p, p, p, p]
    return lib


class PythonPolicy:
    """The reference's host policy, key by key, in float32 where it is float32."""

    def __init__(self, sets, sentinel=-1):
        self.sets, self.sentinel = sets, sentinel
        self.tags = np.full((sets, 8), sentinel, np.int64)
        self.counters = np.zeros((sets, 8), np.float32)
        self.ts = np.zeros(sets, np.int64)
        self.now = 0

    def way_of(self, key, s):
        for j in range(8):
            stored = (int(self.tags[s, j]) * self.sets + s) & 0xFFFFFFFFFFFFFFFF
            if stored == (key & 0xFFFFFFFFFFFFFFFF):
                return j
        return -1

    def insert(self, order, n, max_entries):
        """order: (key, count, first position) of the distinct keys, in histogram order."""
        self.now += 1
        taken, out = set(), []
        for key, count, first in order:
            if len(taken) >= max_entries:
                break
            priority = np.float32(count) / np.float32(n)
            s = (key & 0xFFFFFFFFFFFFFFFF) % self.sets
            if self.ts[s] != self.now:
                factor = np.float32(math.pow(float(DECAY), float(self.now - self.ts[s])))
                self.counters[s] = self.counters[s] * factor
                self.ts[s] = self.now
            hit = self.way_of(key, s)
            if hit >= 0:
                self.counters[s, hit] = self.counters[s, hit] + priority
                continue
            victim = int(np.argmin(self.counters[s]))
            if self.counters[s, victim] > priority:
                continue
            line = s * 8 + victim
            if line in taken:
                continue
            taken.add(line)
            self.counters[s, victim] = priority
            tag = (key & 0xFFFFFFFFFFFFFFFF) // self.sets
            self.tags[s, victim] = np.int64(np.uint64(tag).astype(np.int64)) if tag >= 2 ** 63 else tag
            out.append((line, int(self.tags[s, victim]), first))
        return out


def zipf_batch(rng, n, vocab, negative=False):
    ranks = np.minimum(rng.zipf(1.3, n), vocab) - 1
    keys = (ranks * 7919 + 13) % (vocab * 11)
    if negative:
        keys = keys - vocab * 3            # a share of the keys below zero
    return keys.astype(np.int64)


def state_of(shim, handle, sets):
    tags = np.zeros((sets, 8), np.int64)
    counters = np.zeros((sets, 8), np.float32)
    ts = np.zeros(sets, np.int64)
    shim.hp_state(handle, tags.ctypes.data, counters.ctypes.data, ts.ctypes.data)
    return tags, counters, ts


@pytest.mark.parametrize("sets,max_entries,negative", [(1, 1 << 20, False), (5, 1 << 20, False), (37, 40, False),
                                                       (64, 1 << 20, True)])
def test_inserts_follow_the_reference_policy(shim, sets, max_entries, negative):
    rng = np.random.default_rng(sets)
    handle = shim.hp_create(sets, -1)
    py = PythonPolicy(sets)
    for step in range(8):
        n = [300, 17, 1000, 1, 64, 2000, 5, 800][step]
        keys = zipf_batch(rng, n, 400, negative)
        # histogram: a permutation of the distinct keys, counts falling, first positions right
        hk, hc, hf = np.zeros(n, np.int64), np.zeros(n, np.float32), np.zeros(n, np.int64)
        bins = shim.hp_histogram(keys.ctypes.data, n, hk.ctypes.data, hc.ctypes.data, hf.ctypes.data)
        uniq, first_pos, counts = np.unique(keys, return_index=True, return_counts=True)
        assert bins == uniq.size and sorted(hk[:bins].tolist()) == uniq.tolist()
        assert np.all(np.diff(hc[:bins]) <= 0)
        where = {int(k): (int(c), int(f)) for k, c, f in zip(uniq, counts, first_pos)}
        assert all(where[int(k)] == (int(c), int(f)) for k, c, f in zip(hk[:bins], hc[:bins], hf[:bins]))
        order = [(int(k), int(c), int(f)) for k, c, f in zip(hk[:bins], hc[:bins], hf[:bins])]
        want = py.insert(order, n, max_entries)
        lines, tags, rows = np.zeros(n, np.uint64), np.zeros(n, np.int64), np.zeros(n, np.int64)
        got_n = shim.hp_insert(handle, keys.ctypes.data, n, float(DECAY), max_entries, lines.ctypes.data,
                               tags.ctypes.data, rows.ctypes.data)
        got = list(zip(lines[:got_n].tolist(), tags[:got_n].tolist(), rows[:got_n].tolist()))
        assert got == want, f"insert {step}"
        assert got_n <= max_entries
        t, c, ts = state_of(shim, handle, sets)
        assert np.array_equal(t, py.tags) and np.array_equal(ts, py.ts)
        assert np.array_equal(c.view(np.uint32), py.counters.view(np.uint32)), f"counters after insert {step}"
    shim.hp_destroy(handle)


def test_resident_search_and_invalidate(shim):
    sets = 16
    rng = np.random.default_rng(3)
    handle = shim.hp_create(sets, -1)
    keys = rng.permutation(2000)[:100].astype(np.int64)
    n = keys.size
    buf = [np.zeros(n, np.uint64), np.zeros(n, np.int64), np.zeros(n, np.int64)]
    inserted = shim.hp_insert(handle, keys.ctypes.data, n, float(DECAY), 1 << 20, *(b.ctypes.data for b in buf))
    tags, _, _ = state_of(shim, handle, sets)
    resident = {int(tags[s, w]) * sets + s: s * 8 + w for s in range(sets) for w in range(8) if tags[s, w] != -1}
    assert len(resident) == inserted
    probe = np.concatenate([keys[:40], np.arange(5000, 5020)]).astype(np.int64)
    lines, rows = np.zeros(probe.size, np.uint64), np.zeros(probe.size, np.int64)
    found = shim.hp_find_resident(handle, probe.ctypes.data, probe.size, 1 << 20, lines.ctypes.data, rows.ctypes.data)
    want = [(resident[int(k)], i) for i, k in enumerate(probe) if int(k) in resident]
    assert list(zip(lines[:found].tolist(), rows[:found].tolist())) == want
    capped = shim.hp_find_resident(handle, probe.ctypes.data, probe.size, 3, lines.ctypes.data, rows.ctypes.data)
    assert capped == min(3, len(want))
    gone = np.array([k for k in keys[:40] if int(k) in resident][:10], np.int64)
    cleared = shim.hp_invalidate(handle, gone.ctypes.data, gone.size, lines.ctypes.data)
    assert sorted(lines[:cleared].tolist()) == sorted(resident[int(k)] for k in gone)
    tags2, _, _ = state_of(shim, handle, sets)
    assert (tags2.ravel()[lines[:cleared].astype(np.int64)] == -1).all()
    assert shim.hp_invalidate(handle, gone.ctypes.data, gone.size, lines.ctypes.data) == 0
    shim.hp_destroy(handle)
