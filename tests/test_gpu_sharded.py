"""GPU checks of the row-sharded table: the routing kernels against numpy, the full lookup at
world size 1 against the oracle, and (when the box has at least 2 GPUs) 2-rank runs of every form:
the exchange form over the library's own NCCL communicator, the peer form over symmetric memory,
each with and without hot rows, and the peer form with the cache in front."""
import ctypes as C
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from nv_embedding_cache_b200 import capi, datagen as dg
from nve_helpers import to_dev

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_route_localise_expand_against_numpy(torch_cuda):
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import CudaStages
    for world in (1, 2, 3, 8):
        n, rows = 20000, 100000
        st = CudaStages(n, world)
        keys = dg.zipf_keys(n, rows, 1.05, world, dg.permutation(rows))
        d_keys = to_dev(torch, keys)
        send_keys, send_counts = st.dedup_and_route(d_keys)      # nothing read back yet
        uniq = np.unique(keys)
        u = int(send_counts.sum().item())
        assert u == uniq.size
        owner = uniq % world
        order = np.argsort(owner, kind="stable")
        assert np.array_equal(send_keys[:u].cpu().numpy(), uniq[order])
        assert np.array_equal(send_counts.cpu().numpy(), np.bincount(owner, minlength=world))
        slot = np.empty(u, np.int64)
        slot[order] = np.arange(u)
        assert np.array_equal(st.slot_of_unique[:u].cpu().numpy(), slot)
        # expand: position i -> slot of its unique key
        capi.check(capi.lib.nve_b200_shard_expand_slots(
            capi.KEY_INT64, st.inverse.data_ptr(), st.offsets.data_ptr(), st.slot_of_unique.data_ptr(),
            st.num_unique_dev, n, st.slot_of_position.data_ptr(), None))
        torch.cuda.synchronize()
        assert np.array_equal(st.slot_of_position[:n].cpu().numpy(), slot[np.searchsorted(uniq, keys)])
        k2 = d_keys.clone()
        capi.check(capi.lib.nve_b200_shard_localise(capi.KEY_INT64, k2.data_ptr(), n, world, None))
        torch.cuda.synchronize()
        assert np.array_equal(k2.cpu().numpy(), keys // world)
        st.close()


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_world_size_one_matches_oracle(torch_cuda, oracle, dtype):
    torch = torch_cuda
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
    rows, dim = 50000, 64
    npdt = np.float16 if dtype == "f16" else np.float32
    table = dg.normal_table(rows, dim, 0.02, 3, npdt)
    t = ShardedEmbeddingTable(to_dev(torch, table), max_keys=1 << 16)
    keys = dg.zipf_keys(4096 * 8, rows, 1.05, 5, dg.permutation(rows))
    out = t.lookup_pooled(to_dev(torch, keys), "sum", fixed_hotness=8)
    torch.cuda.synchronize()
    want = oracle.lookup_pooled(table.view(np.uint8).reshape(rows, -1), dtype, dim, keys, "sum",
                                hotness=8, out_dtype=dtype)
    assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8))
    _, offs = dg.csr_bags(3000, 0, 20, 6)
    keys = dg.uniform_keys(int(offs[-1]), rows, 7)
    out = t.lookup_pooled(to_dev(torch, keys), "mean", csr_offsets=to_dev(torch, offs))
    torch.cuda.synchronize()
    want = oracle.lookup_pooled(table.view(np.uint8).reshape(rows, -1), dtype, dim, keys, "mean",
                                offsets=offs, out_dtype=dtype)
    assert np.array_equal(out.cpu().numpy().view(np.uint8), want.view(np.uint8))
    t.close()


WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NVE_ROOT"])
from nv_embedding_cache_b200 import datagen as dg
from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
rows_per_rank, dim = 40000, 64
total = rows_per_rank * world
table = dg.dyadic_table(total, dim, 3, np.float16)
mode = os.environ.get("NVE_TEST_SHARD_MODE", "alltoall")
if mode.startswith("peer"):
    from nv_embedding_cache_b200.sharded import allocate_symmetric_shard
    shard = allocate_symmetric_shard(rows_per_rank, dim, torch.float16)
    shard.copy_(torch.from_numpy(table[rank::world].copy()))
else:
    shard = torch.from_numpy(table[rank::world].copy()).cuda()
cached = mode == "peer_cached"
hot = mode.endswith("_hot")
mode = mode.split("_")[0]
t = ShardedEmbeddingTable(shard, max_keys=1 << 16, mode=mode, hot_rows=3000 if hot else 0,
                          cache_bytes=(2000 // 8) * (64 + 8 * dim * 2 + 32) if cached else 0)
if hot:     # the rows a sample of the key stream asks for most are replicated on every rank
    sample = np.concatenate([dg.zipf_keys(8192, total, 1.05, 300 + b + rank, dg.permutation(total)) for b in range(3)])
    assert 0 < t.set_hot_keys(torch.from_numpy(sample).cuda()) <= 3000
ok = True
hits = 0
for step in range(3):
    keys = dg.zipf_keys(2048 * 8, total, 1.05, 100 + 10 * step + rank, dg.permutation(total))
    if cached:      # rows of an earlier batch are resident: some keys are served locally, results identical
        t.populate_cache(torch.from_numpy(dg.zipf_keys(4096, total, 1.05, 50 + step + rank, dg.permutation(total))).cuda())
        t.cache_misses(reset=True)
    out = t.lookup_pooled(torch.from_numpy(keys).cuda(), "sum", fixed_hotness=8)
    torch.cuda.synchronize()
    if cached:
        hits += keys.size - t.cache_misses(reset=True)
    want = table[keys].astype(np.float32).reshape(2048, 8, dim).sum(1).astype(np.float16)
    ok = ok and bool(np.array_equal(out.cpu().numpy(), want))
if cached:
    ok = ok and hits > 1000
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
t.close()
dist.barrier()
dist.destroy_process_group()
sys.exit(0 if int(flag.item()) == 1 else 3)
'''


@pytest.mark.parametrize("mode", ["alltoall", "alltoall_hot", "peer", "peer_hot", "peer_cached"])
def test_two_ranks_nccl(torch_cuda, tmp_path, mode):
    torch = torch_cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NVE_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0", NVE_TEST_SHARD_MODE=mode)
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                          "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port",
                          str(port), str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


LEAVER = r'''
import os, sys
from datetime import timedelta
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NVE_ROOT"])
from nv_embedding_cache_b200 import datagen as dg
from nv_embedding_cache_b200.sharded import PeerLeft, PeerMonitor, ShardedEmbeddingTable
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
store = dist.TCPStore("127.0.0.1", int(os.environ["NVE_STORE_PORT"]), world, rank == 0, timeout=timedelta(seconds=60))
dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=timedelta(seconds=60))
rows_per_rank, dim = 20000, 32
total = rows_per_rank * world
table = dg.dyadic_table(total, dim, 3, np.float16)
monitor = PeerMonitor(store, rank, world)
t = ShardedEmbeddingTable(torch.from_numpy(table[rank::world].copy()).cuda(), max_keys=1 << 14, mode="alltoall",
                          monitor=monitor)
keys = torch.from_numpy(dg.zipf_keys(1024 * 8, total, 1.05, 9 + rank, dg.permutation(total))).cuda()
out = t.lookup_pooled(keys, "sum", fixed_hotness=8)
torch.cuda.synchronize()
want = table[keys.cpu().numpy()].astype(np.float32).reshape(1024, 8, dim).sum(1).astype(np.float16)
ok = bool(np.array_equal(out.cpu().numpy(), want))
dist.barrier()
torch.cuda.synchronize()                 # the step is over: nothing of this rank is in flight
if rank == world - 1:
    monitor.announce_leave()
    os._exit(0 if ok else 3)
store.wait([monitor._key(world - 1)], timedelta(seconds=30))
try:
    t.lookup_pooled(keys, "sum", fixed_hotness=8)
    code = 4                              # a lookup that needs the departed rank must not be attempted
except PeerLeft:
    code = 0 if ok else 3
os._exit(code)
'''


def test_rank_leaves_between_steps_nccl(torch_cuda, tmp_path):
    """A rank leaves between two steps with nothing in flight and says so on the store; the other
    rank learns of it on the host and refuses its next lookup before any kernel or collective is
    launched.  NVLS is off and the exchange form is used (no peer-mapped memory involved)."""
    torch = torch_cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "leaver.py"
    script.write_text(LEAVER)
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    procs = []
    for rank in range(2):
        env = dict(os.environ, NVE_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0", RANK=str(rank), WORLD_SIZE="2",
                   LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(ports[0]),
                   NVE_STORE_PORT=str(ports[1]))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert [p.returncode for p in procs] == [0, 0], "\n".join(o[-1500:] for o in outs)
