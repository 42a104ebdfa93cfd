"""GPU checks of the row-sharded table object (nve_b200_sharded_table_*) on ONE GPU: the shards of
every rank live on the same device, one table object per emulated rank.  The peer form gets all
shard addresses; the exchange form runs its ranks as threads of this process over an in-process
transport (the caller-supplied exchange_ops), so the whole C++ path — hash de-duplication, owner
bucketing, the two exchanges, row service, pooling, hot rows — is compared with the oracle at world
sizes 1, 2, 3 and 8 without a second GPU."""
import ctypes as C
import threading
import traceback

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import to_dev

pytestmark = pytest.mark.gpu


def make_shards(torch, table, world):
    return [to_dev(torch, table[r::world].copy()) for r in range(world)]


class Loopback:
    """All-gather and all-to-all among the threads of one process: every rank publishes its send
    buffer, the ranks meet at a barrier, and each copies its part out of the others' buffers."""

    def __init__(self, world, fail_at=None, stall=None):
        self.world = world
        self.barrier = threading.Barrier(world)
        self.slots = [None] * world
        self.fail_at = fail_at          # (rank, call number): that call reports an error
        self.stall = stall              # torch module: the all-gather leaves a long kernel on the stream
        self.calls = [0] * world

    @staticmethod
    def _copy(dst, src, nbytes):
        from cuda import cudart
        if nbytes:
            (err,) = cudart.cudaMemcpy(dst, src, nbytes, cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice)
            assert int(err) == 0, err

    @staticmethod
    def _sync():
        from cuda import cudart
        (err,) = cudart.cudaDeviceSynchronize()
        assert int(err) == 0, err

    def ops(self, rank):
        def all_gather(user, d_in, d_out, count, stream):
            try:
                self.calls[rank] += 1
                if self.fail_at == (rank, self.calls[rank]):
                    return 7
                if self.stall is not None:
                    self.stall.cuda._sleep(int(3e9))       # about 1.5 s of GPU time, then the stream goes on
                    return 0
                self._sync()
                self.slots[rank] = d_in
                self.barrier.wait(timeout=20)
                for r in range(self.world):
                    self._copy(d_out + r * count * 4, self.slots[r], count * 4)
                self._sync()
                self.barrier.wait(timeout=20)
                return 0
            except Exception:       # noqa: BLE001 - reported to the library as a transport error
                traceback.print_exc()
                return 1

        def all_to_all(user, d_send, send_counts, d_recv, recv_counts, elem_bytes, stream):
            try:
                self._sync()
                mine = [send_counts[p] for p in range(self.world)]
                self.slots[rank] = (d_send, mine)
                self.barrier.wait(timeout=20)
                at = 0
                for p in range(self.world):
                    src, counts = self.slots[p]
                    assert counts[rank] == recv_counts[p]
                    self._copy(d_recv + at * elem_bytes, src + sum(counts[:rank]) * elem_bytes,
                               counts[rank] * elem_bytes)
                    at += recv_counts[p]
                self._sync()
                self.barrier.wait(timeout=20)
                return 0
            except Exception:       # noqa: BLE001
                traceback.print_exc()
                return 1

        o = capi.ExchangeOps()
        o.user = None
        o.all_gather_u32 = capi.ALL_GATHER_U32_FN(all_gather)
        o.all_to_all_v = capi.ALL_TO_ALL_V_FN(all_to_all)
        return o


def run_ranks(world, fn):
    """fn(rank) on one thread per rank; re-raises the first failure."""
    errors = [None] * world
    results = [None] * world

    def body(r):
        try:
            results[r] = fn(r)
        except BaseException as e:      # noqa: BLE001
            traceback.print_exc()
            errors[r] = e
    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    for e in errors:
        if e is not None:
            raise e
    return results


def expected(oracle, table, dtype, keys, pooling, *, hotness=0, offsets=None, default_row=-1, weights=None):
    rows, dim = table.shape
    return oracle.lookup_pooled(table.view(np.uint8).reshape(rows, -1), dtype, dim, keys, pooling,
                                hotness=hotness, offsets=offsets, out_dtype=dtype, default_row=default_row,
                                weights=weights)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("dtype,npdt", [("f16", np.float16), ("f32", np.float32)])
def test_peer_form_with_and_without_hot_rows(torch_cuda, oracle, world, dtype, npdt):
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
    rows_per_rank, dim = 6000, 64
    total = rows_per_rank * world
    table = dg.normal_table(total, dim, 0.02, 3, npdt)
    shards = make_shards(torch, table, world)
    ptrs = [s.data_ptr() for s in shards]
    perm = dg.permutation(total)
    sample = to_dev(torch, np.concatenate([dg.zipf_keys(8192, total, 1.05, 50 + b, perm) for b in range(4)]))
    for rank in range(world):
        t = ShardedEmbeddingTable(shards[rank], max_keys=1 << 16, mode="peer", world=world, rank=rank,
                                  peer_shards=ptrs, hot_rows=3000, default_row=5)
        keys = dg.zipf_keys(2048 * 8, total, 1.05, 100 + rank, perm)
        keys[::41] = -7                 # read the default row
        keys[3::53] = total + 11
        _, offs = dg.csr_bags(700, 0, 40, 6 + rank)
        ckeys = dg.uniform_keys(int(offs[-1]), total, 7 + rank)
        w = np.random.default_rng(8).uniform(-1, 1, ckeys.size).astype(np.float32)
        for hot in (False, True):
            if hot:
                assert 0 < t.set_hot_keys(sample) <= 3000
            out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
            torch.cuda.synchronize()
            want = expected(oracle, table, dtype, keys, "sum", hotness=8, default_row=5)
            assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8)), (rank, hot)
            out = t.lookup_pooled(to_dev(torch, ckeys), "mean", csr_offsets=to_dev(torch, offs))
            torch.cuda.synchronize()
            want = expected(oracle, table, dtype, ckeys, "mean", offsets=offs, default_row=5)
            assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8)), (rank, hot)
            out = t.lookup_pooled(to_dev(torch, ckeys), "weighted_sum", csr_offsets=to_dev(torch, offs),
                                  weights=to_dev(torch, w))
            torch.cuda.synchronize()
            want = expected(oracle, table, dtype, ckeys, "wsum", offsets=offs, default_row=5, weights=w)
            assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8)), (rank, hot)
            # fixed hotness below the lane-group size, mean and weighted mean (the pipelined kernel)
            fkeys = keys[:2000 * 5]
            fw = np.random.default_rng(9).uniform(0.1, 1, fkeys.size).astype(np.float32)
            for pooling, ref_pool, weights in (("mean", "mean", None), ("weighted_mean", "wmean", fw)):
                out = t.lookup_pooled(to_dev(torch, fkeys), pooling, fixed_hotness=5,
                                      weights=None if weights is None else to_dev(torch, weights))
                torch.cuda.synchronize()
                want = expected(oracle, table, dtype, fkeys, ref_pool, hotness=5, default_row=5, weights=weights)
                assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8)), (rank, hot, pooling)
        t.close()


def test_hot_rows_choice_and_refresh(torch_cuda, oracle):
    """More distinct keys in the sample than hot rows: the most frequent ones are kept; keys that are
    no rows of the table are ignored; an empty sample empties the hot table; results never change."""
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
    world, rows_per_rank, dim = 4, 5000, 32
    total = world * rows_per_rank
    table = dg.dyadic_table(total, dim, 3, np.float16)
    shards = make_shards(torch, table, world)
    t = ShardedEmbeddingTable(shards[1], max_keys=1 << 15, mode="peer", world=world, rank=1,
                              peer_shards=[s.data_ptr() for s in shards], hot_rows=64)
    hot = np.arange(100, 164, dtype=np.int64) * 7 % total        # 64 distinct rows, five times each
    sample = np.concatenate([np.repeat(hot, 5), dg.uniform_keys(3000, total, 1),
                             np.array([-1, -9, total, total + 5], np.int64)])
    assert t.set_hot_keys(to_dev(torch, sample)) == 64
    keys = np.concatenate([np.repeat(hot, 3), dg.uniform_keys(64 * 5, total, 2)])
    out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
    torch.cuda.synchronize()
    want = expected(oracle, table, "f16", keys, "sum", hotness=8)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    # the copies are a snapshot: after the shards change, a refresh brings the new rows in
    for s in shards:
        s.mul_(2)
    assert t.set_hot_keys(to_dev(torch, np.repeat(hot, 2))) == 64
    out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
    torch.cuda.synchronize()
    want2 = expected(oracle, (table * np.float16(2)).astype(np.float16), "f16", keys, "sum", hotness=8)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want2.view(np.uint16))
    assert t.set_hot_keys(torch.empty(0, dtype=torch.int64, device="cuda")) == 0
    out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want2.view(np.uint16))
    t.close()


@pytest.mark.parametrize("mode", ["peer", "alltoall"])
def test_padded_shard_rows_with_hot_rows(torch_cuda, oracle, mode):
    """Shard rows stored with padding (128-byte rows at a 144-byte stride): the hot table and the
    exchange buffers keep their own, packed stride."""
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
    world, rows_per_rank, dim = (3, 4000, 64) if mode == "peer" else (1, 12000, 64)
    total = world * rows_per_rank
    table = dg.normal_table(total, dim, 0.02, 5, np.float16)
    shards = []
    for r in range(world):
        wide = torch.zeros((rows_per_rank, dim + 8), dtype=torch.float16, device="cuda")
        wide[:, :dim] = to_dev(torch, table[r::world].copy())
        shards.append(wide[:, :dim])                      # stride 72 elements = 144 bytes
    assert shards[0].stride(0) == dim + 8
    t = ShardedEmbeddingTable(shards[0], max_keys=1 << 14, mode=mode, world=world, rank=0,
                              peer_shards=[s.data_ptr() for s in shards] if mode == "peer" else None,
                              hot_rows=1500)
    perm = dg.permutation(total)
    assert t.set_hot_keys(to_dev(torch, dg.zipf_keys(20000, total, 1.05, 3, perm))) == 1500
    keys = dg.zipf_keys(1500 * 8, total, 1.05, 4, perm)
    out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
    torch.cuda.synchronize()
    want = expected(oracle, table, "f16", keys, "sum", hotness=8)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    t.close()


@pytest.mark.parametrize("hot_rows", [0, 2000])
@pytest.mark.parametrize("dtype,npdt", [("f16", np.float16), ("f32", np.float32)])
def test_exchange_form_world_one(torch_cuda, oracle, dtype, npdt, hot_rows):
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
    rows, dim = 50000, 64
    table = dg.normal_table(rows, dim, 0.02, 3, npdt)
    t = ShardedEmbeddingTable(to_dev(torch, table), max_keys=1 << 16, mode="alltoall", world=1, rank=0,
                              hot_rows=hot_rows)
    perm = dg.permutation(rows)
    if hot_rows:
        assert t.set_hot_keys(to_dev(torch, dg.zipf_keys(30000, rows, 1.05, 4, perm))) == hot_rows
    keys = dg.zipf_keys(4096 * 8, rows, 1.05, 5, perm)
    out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
    torch.cuda.synchronize()
    want = expected(oracle, table, dtype, keys, "sum", hotness=8)
    assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8))
    _, offs = dg.csr_bags(3000, 0, 20, 6)
    keys = dg.uniform_keys(int(offs[-1]), rows, 7)
    out = t.lookup_pooled(to_dev(torch, keys), "mean", csr_offsets=to_dev(torch, offs.astype(np.int32)))
    torch.cuda.synchronize()
    want = expected(oracle, table, dtype, keys, "mean", offsets=offs)
    assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8))
    t.close()


@pytest.mark.parametrize("world,hot_rows", [(2, 0), (3, 1500), (8, 0), (8, 4000)])
def test_exchange_form_ranks_as_threads(torch_cuda, oracle, world, hot_rows):
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
    rows_per_rank, dim = 4000, 64
    total = rows_per_rank * world
    table = dg.dyadic_table(total, dim, 3, np.float16)
    shards = make_shards(torch, table, world)
    perm = dg.permutation(total)
    net = Loopback(world)
    transports = [net.ops(r) for r in range(world)]
    max_keys = 2048             # 4000 hot rows come through the exchange in two rounds

    def rank_body(rank):
        torch.cuda.set_device(0)
        t = ShardedEmbeddingTable(shards[rank], max_keys=max_keys, mode="alltoall", world=world, rank=rank,
                                  transport=transports[rank], hot_rows=hot_rows, timeout_ms=60000)
        if hot_rows:
            sample = np.concatenate([dg.zipf_keys(8192, total, 1.05, 50 + b + rank, perm) for b in range(3)])
            assert 0 < t.set_hot_keys(to_dev(torch, sample)) <= hot_rows
        seen = []
        for step in range(3):
            # rank 1 sends an empty batch in step 1: it still serves the others
            n = 0 if (rank == 1 and step == 1) else 256 * 8
            keys = dg.zipf_keys(n, total, 1.05, 100 + 10 * step + rank, perm) if n else np.zeros(0, np.int64)
            out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
            torch.cuda.synchronize()
            if n:
                want = expected(oracle, table, "f16", keys, "sum", hotness=8)
                assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16)), (rank, step)
            seen.append((np.unique(keys).size, dict(t.last_exchange)))
        t.close()
        return seen

    results = run_ranks(world, rank_body)
    for rank, seen in enumerate(results):
        for uniq, ex in seen:
            assert ex["unique"] <= uniq                      # hot keys take no part in the exchange
            if not hot_rows:
                assert ex["unique"] == uniq
    # every key a rank sent was served by somebody
    for step in range(3):
        assert sum(r[step][1]["unique"] for r in results) == sum(r[step][1]["served"] for r in results)


def test_exchange_failure_is_reported_and_remembered(torch_cuda):
    """A transport call that fails ends the lookup with ExchangeFailed (NVE_ERROR_RUNTIME underneath);
    the table then refuses further lookups.  A host wait that outlasts exchange_timeout_ms does the
    same: here the transport leaves a kernel of about 1.5 s on the stream (bounded; nothing hangs)."""
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ExchangeFailed, ShardedEmbeddingTable
    world, rows_per_rank, dim = 2, 2000, 32
    total = world * rows_per_rank
    table = dg.dyadic_table(total, dim, 3, np.float16)
    shards = make_shards(torch, table, world)
    keys = to_dev(torch, dg.uniform_keys(256 * 8, total, 3))

    net = Loopback(world, fail_at=(0, 1))
    ops0 = net.ops(0)
    t = ShardedEmbeddingTable(shards[0], max_keys=1 << 12, mode="alltoall", world=world, rank=0, transport=ops0)
    with pytest.raises(ExchangeFailed):
        t.lookup_pooled(keys, "sum", fixed_hotness=8)
    with pytest.raises(ExchangeFailed):
        t.lookup_pooled(keys, "sum", fixed_hotness=8)
    t.close()

    net = Loopback(world, stall=torch)
    ops0 = net.ops(0)
    t = ShardedEmbeddingTable(shards[0], max_keys=1 << 12, mode="alltoall", world=world, rank=0, transport=ops0,
                              timeout_ms=200)
    with pytest.raises(ExchangeFailed) as e:
        t.lookup_pooled(keys, "sum", fixed_hotness=8)
    assert "did not complete" in str(e.value)
    torch.cuda.synchronize()            # the bounded kernel ends by itself
    t.close()


def test_c5_batch_size_on_one_gpu(torch_cuda, oracle):
    """The sharded configuration's batch (131 072 bags x 8 keys, Zipf 1.05) at world sizes 1 and 8 with
    the table scaled down in rows: peer form with hot rows, and the exchange form at world size 1."""
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
    bags, hot, dim = 131_072, 8, 64
    n = bags * hot
    for world, rows_per_rank in ((1, 8_000_000), (8, 1_000_000)):
        total = world * rows_per_rank
        gen = torch.Generator(device="cuda")
        gen.manual_seed(60)
        full = (torch.randn((total, dim), generator=gen, device="cuda") * 0.02).half()
        shards = [full[r::world].contiguous() for r in range(world)]
        keys = dg.zipf_keys(n, total, 1.05, 600)
        uniq, inv = np.unique(keys, return_inverse=True)
        mirror = full[torch.from_numpy(uniq).cuda()].cpu().numpy()
        want = oracle.lookup_pooled(mirror.view(np.uint8).reshape(uniq.size, -1), "f16", dim,
                                    inv.astype(np.int64), "sum", hotness=hot, out_dtype="f16")
        d_keys = to_dev(torch, keys)
        sample = to_dev(torch, np.concatenate([dg.zipf_keys(n, total, 1.05, 700 + b) for b in range(3)]))
        t = ShardedEmbeddingTable(shards[0], max_keys=n, mode="peer", world=world, rank=0,
                                  peer_shards=[s.data_ptr() for s in shards], hot_rows=1 << 20)
        for use_hot in (False, True):
            if use_hot:
                assert t.set_hot_keys(sample) > 100_000
            out = t.lookup_pooled(d_keys, "sum", fixed_hotness=hot)
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16)), (world, use_hot)
        t.close()
        if world == 1:
            t = ShardedEmbeddingTable(shards[0], max_keys=n, mode="alltoall", world=1, rank=0)
            out = t.lookup_pooled(d_keys, "sum", fixed_hotness=hot)
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
            t.close()
        del full, shards
