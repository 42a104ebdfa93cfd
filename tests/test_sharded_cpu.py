"""World-size-2 and -3 runs of the sharded-table exchange protocol on CPU (gloo): the split sizes,
ordering and index maps of nv_embedding_cache_b200.sharded.ShardedEmbeddingTable, with the device
stages replaced by a host implementation of the same stage interface.  The result must equal a
plain pooled lookup in the unsharded table."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nv_embedding_cache_b200 import datagen as dg


class HostStages:
    """numpy restatement of the stage interface (test infrastructure only)."""

    def __init__(self, world):
        self.world = world

    def dedup_and_route(self, keys):
        k = keys.numpy()
        self.unique, self.inv = np.unique(k, return_inverse=True)
        owner = (self.unique.astype(np.uint64) % np.uint64(self.world)).astype(np.int64)
        order = np.argsort(owner, kind="stable")
        self.slot_of_unique = np.empty_like(order)
        self.slot_of_unique[order] = np.arange(order.size)
        counts = np.bincount(owner, minlength=self.world).astype(np.int64)
        return torch.from_numpy(self.unique[order].copy()), torch.from_numpy(counts)

    def serve(self, shard, recv_keys):
        local = (recv_keys.numpy().astype(np.uint64) // np.uint64(self.world)).astype(np.int64)
        return shard[torch.from_numpy(local)]

    def pool(self, rows, n, pooling, hotness, offsets, out):
        r = rows.numpy()[self.slot_of_unique[self.inv]].astype(np.float32)
        if offsets is None:
            offs = np.arange(0, n + 1, hotness)
        else:
            offs = offsets.numpy()
        for b in range(offs.size - 1):
            acc = np.zeros(r.shape[1], np.float32)
            for i in range(offs[b], offs[b + 1]):
                acc = acc + r[i]
            out[b] = torch.from_numpy(acc.astype(out.numpy().dtype))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows_per_rank, dim, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
        total = rows_per_rank * world
        table = dg.dyadic_table(total, dim, 3, np.float32)
        shard = torch.from_numpy(table[rank::world].copy())
        t = ShardedEmbeddingTable(shard, max_keys=4096, stages=HostStages(world))
        keys = dg.zipf_keys(64 * 8, total, 1.05, 100 + rank, dg.permutation(total))
        out = t.lookup_pooled(torch.from_numpy(keys), "sum", fixed_hotness=8)
        want = table[keys].reshape(64, 8, dim).sum(1)
        ok_fixed = bool(np.array_equal(out.numpy(), want))
        _, offs = dg.csr_bags(40, 0, 9, 200 + rank)
        keys2 = dg.uniform_keys(int(offs[-1]), total, 300 + rank)
        out2 = t.lookup_pooled(torch.from_numpy(keys2), "sum", csr_offsets=torch.from_numpy(offs))
        want2 = np.stack([table[keys2[offs[b]:offs[b + 1]]].sum(0) if offs[b + 1] > offs[b]
                          else np.zeros(dim, np.float32) for b in range(40)])
        ok_csr = bool(np.array_equal(out2.numpy(), want2))
        q.put((rank, ok_fixed, ok_csr, t.last_exchange["unique"], t.last_exchange["served"]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_lookup_matches_unsharded(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 500, 16, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == list(range(world))
    assert all(r[1] and r[2] for r in results), results
    # every unique key requested by some rank is served by exactly one owner
    assert sum(r[3] for r in results) == sum(r[4] for r in results)


def _leaver_worker(rank, world, pg_port, store_port, announce, q):
    """Every rank does one lookup; the last rank then leaves (announced on the store, or silently);
    the others try a second lookup and report how it ended."""
    from datetime import timedelta
    store = dist.TCPStore("127.0.0.1", store_port, world, rank == 0, timeout=timedelta(seconds=60))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(pg_port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=8))
    from nv_embedding_cache_b200.sharded import ExchangeFailed, PeerLeft, PeerMonitor, ShardedEmbeddingTable
    total, dim = 300 * world, 8
    table = dg.dyadic_table(total, dim, 3, np.float32)
    monitor = PeerMonitor(store, rank, world)
    t = ShardedEmbeddingTable(torch.from_numpy(table[rank::world].copy()), max_keys=1024,
                              stages=HostStages(world), monitor=monitor)
    keys = torch.from_numpy(dg.uniform_keys(64, total, 7 + rank))
    out = t.lookup_pooled(keys, "sum", fixed_hotness=8)
    first_ok = bool(np.array_equal(out.numpy(), table[keys.numpy()].reshape(8, 8, dim).sum(1)))
    dist.barrier()                                   # the step is over on every rank
    leaver = world - 1
    if rank == leaver:
        if announce:
            monitor.announce_leave()
        q.put((rank, first_ok, "left"))
        q.close()
        q.join_thread()
        os._exit(0)                                  # gone, without tearing the group down
    if announce:
        store.wait([monitor._key(leaver)], timedelta(seconds=30))    # the news arrives on the host
    outcome = "completed"
    try:
        t.lookup_pooled(keys, "sum", fixed_hotness=8)
    except PeerLeft:
        outcome = "peer_left"
    except ExchangeFailed:
        outcome = "exchange_failed"
        try:
            t.lookup_pooled(keys, "sum", fixed_hotness=8)       # refused at once from now on
            outcome = "second_lookup_completed"
        except ExchangeFailed:
            pass
    q.put((rank, first_ok, outcome))
    q.close()
    q.join_thread()
    os._exit(0)


@pytest.mark.parametrize("announce,expected", [(True, "peer_left"), (False, "exchange_failed")])
def test_a_rank_that_leaves_between_steps(announce, expected):
    """Failure detection without any device fault: a rank leaves between two steps.  Announced on
    the store, the others refuse their next lookup on the host before any collective; unannounced,
    the process group's short timeout (or the closed connection) ends the collective with an error
    that the table reports and remembers."""
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ports = (_free_port(), _free_port())
    procs = [ctx.Process(target=_leaver_worker, args=(r, world, ports[0], ports[1], announce, q))
             for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert all(r[1] for r in results), results
    assert results[world - 1][2] == "left"
    assert [r[2] for r in results[:world - 1]] == [expected] * (world - 1), results
