"""Row-sharded embedding table over several GPUs, one process per GPU.

Row ``r`` of the global table lives on rank ``r mod W`` at local index ``r // W``.  Two ways to
serve a pooled lookup:

``mode="peer"`` (the one to use on NVLink): every rank allocates its shard in symmetric memory, the
ranks exchange the mapped base addresses once, and the fused lookup kernel of libnve_b200
(``nve_b200_lookup_pool`` with ``shard_tables``) reads each row straight from its owner's HBM — no
collective and no host synchronisation on the lookup path.  This is what the reference does with
one address range mapped over all shards (src/distributed.cpp:155-256, src/memblock_nvl.cpp:40-119).
``cache_bytes`` adds the set-associative cache in front of the peer reads.

``mode="alltoall"`` (any process group):

    dedup keys -> bucket unique keys by owner -> all-to-all (counts, keys)
    -> owners gather their rows -> all-to-all (rows) -> pool from the received rows

so every distinct row crosses the fabric once per rank and batch, whatever its multiplicity, at the
price of a sort-based dedup, a routing sort and one host read-back (the split sizes) per lookup.
The device stages are kernels of libnve_b200 (``nve_b200_deduper_dedup``, ``nve_b200_shard_route``,
``nve_b200_shard_localise``, ``nve_b200_gather_rows``, ``nve_b200_shard_expand_slots``,
``nve_b200_lookup_pool``); torch.distributed supplies the collectives.  ``stages`` is the object
that runs them: the product uses :class:`CudaStages`; the exchange protocol itself (split sizes,
ordering) is backend-agnostic, which is what the multi-process CPU tests exercise with a host
implementation of the same stage interface.

Results of both modes are those of a lookup in the unsharded table.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import capi


class PeerLeft(RuntimeError):
    """A rank of the group announced that it left: lookups that need it are refused."""


class ExchangeFailed(RuntimeError):
    """A collective of the exchange form ended with an error (a peer died, a timeout ran out).  The
    table refuses further lookups: its process group is no longer usable."""


class PeerMonitor:
    """Membership of the ranks serving a sharded table, kept on the host in a torch.distributed
    store (TCPStore, FileStore, HashStore).  A rank that leaves between two steps, with none of
    its kernels or collectives in flight, calls :meth:`announce_leave`; the others call
    :meth:`check` before they launch their next lookup and get :class:`PeerLeft` instead of a
    collective that can never complete or a read of memory that is gone.  A rank that dies without
    announcing it is caught by the process group's timeout (see :class:`ExchangeFailed`)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "nve_b200/sharded"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/left/{rank}"

    def announce_leave(self) -> None:
        self.store.set(self._key(self.rank), b"1")

    def departed(self):
        return [r for r in range(self.world) if r != self.rank and self.store.check([self._key(r)])]

    def check(self) -> None:
        gone = self.departed()
        if gone:
            raise PeerLeft(f"rank(s) {gone} left the group that serves this table")


def _split_list(t: torch.Tensor):
    return [int(x) for x in t.cpu().tolist()]


class CudaStages:
    """Device stages on the current CUDA device / current stream, through the C ABI."""

    def __init__(self, max_keys: int, world: int):
        self.world = world
        self.max_keys = max_keys
        self.deduper = C.c_void_p()
        capi.check(capi.lib.nve_b200_deduper_create(C.byref(self.deduper), capi.KEY_INT64, -1, max_keys))
        nbytes = C.c_uint64()
        capi.check(capi.lib.nve_b200_shard_route_scratch_bytes(max_keys, C.byref(nbytes)))
        dev = torch.device("cuda", torch.cuda.current_device())
        self.route_scratch = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
        i64 = dict(dtype=torch.int64, device=dev)
        self.unique = torch.empty(max_keys + 1, **i64)
        self.counts = torch.empty(max_keys + 1, **i64)
        self.inverse = torch.empty(max_keys + 1, **i64)
        self.offsets = torch.empty(max_keys + 2, **i64)
        self.send_keys = torch.empty(max_keys + 1, **i64)
        self.slot_of_unique = torch.empty(max_keys + 1, **i64)
        self.slot_of_position = torch.empty(max_keys + 1, **i64)
        self.send_counts = torch.zeros(2 * world, **i64)
        p = C.c_void_p()
        capi.check(capi.lib.nve_b200_deduper_device_num_runs(self.deduper, C.byref(p)))
        self.num_unique_dev = p.value

    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    def dedup_and_route(self, keys: torch.Tensor):
        """-> (send_keys, send_counts[W]): unique keys grouped by owner (the first sum(send_counts)
        entries are valid) and how many go to each rank.  Nothing is read back to the host here."""
        n = keys.numel()
        capi.check(capi.lib.nve_b200_deduper_dedup(
            self.deduper, keys.data_ptr(), n, self.unique.data_ptr(), self.counts.data_ptr(), None,
            None, self.inverse.data_ptr(), self.offsets.data_ptr(), self._stream(), 0))
        capi.check(capi.lib.nve_b200_shard_route(
            capi.KEY_INT64, self.unique.data_ptr(), self.num_unique_dev, max(n, 1), self.world,
            self.send_keys.data_ptr(), self.slot_of_unique.data_ptr(), self.send_counts.data_ptr(),
            self.route_scratch.data_ptr(), self.route_scratch.numel(), self._stream()))
        return self.send_keys, self.send_counts[:self.world]

    def serve(self, shard: torch.Tensor, recv_keys: torch.Tensor) -> torch.Tensor:
        """Rows of the local shard for the received GLOBAL keys (localised in place)."""
        r = recv_keys.numel()
        rows = torch.empty((r, shard.shape[1]), dtype=shard.dtype, device=shard.device)
        if r == 0:
            return rows
        capi.check(capi.lib.nve_b200_shard_localise(capi.KEY_INT64, recv_keys.data_ptr(), r,
                                                    self.world, self._stream()))
        row_bytes = shard.shape[1] * shard.element_size()
        g = capi.GatherArgs()
        g.table = shard.data_ptr()
        g.num_rows = shard.shape[0]
        g.row_stride = shard.stride(0) * shard.element_size()
        g.value_dtype = capi.DTYPE_FLOAT16 if shard.dtype == torch.float16 else capi.DTYPE_FLOAT32
        g.default_row_index = -1
        g.cache = None
        g.key_type = capi.KEY_INT64
        g.keys = recv_keys.data_ptr()
        g.num_keys = r
        g.output = rows.data_ptr()
        g.output_stride = row_bytes
        g.output_dtype = g.value_dtype
        g.row_copy_bytes = row_bytes
        capi.check(capi.lib.nve_b200_gather_rows(C.byref(g), self._stream()))
        return rows

    def pool(self, rows: torch.Tensor, n: int, pooling: int, hotness: int, offsets, out: torch.Tensor):
        capi.check(capi.lib.nve_b200_shard_expand_slots(
            capi.KEY_INT64, self.inverse.data_ptr(), self.offsets.data_ptr(),
            self.slot_of_unique.data_ptr(), self.num_unique_dev, n,
            self.slot_of_position.data_ptr(), self._stream()))
        a = capi.PoolArgs()
        a.table = rows.data_ptr()
        a.num_rows = rows.shape[0]
        a.row_stride = rows.shape[1] * rows.element_size()
        a.value_dtype = capi.DTYPE_FLOAT16 if rows.dtype == torch.float16 else capi.DTYPE_FLOAT32
        a.row_width = rows.shape[1]
        a.default_row_index = -1
        a.cache = None
        a.key_type = capi.KEY_INT64
        a.keys = self.slot_of_position.data_ptr()
        a.num_keys = n
        a.pooling_type = pooling
        a.sparse_type = capi.SPARSE_CSR if offsets is not None else capi.SPARSE_FIXED
        a.csr_offsets = offsets.data_ptr() if offsets is not None else None
        a.offset_bytes = 8
        a.num_bags = (offsets.numel() - 1) if offsets is not None else n // hotness
        a.fixed_hotness = hotness
        a.weights = None
        a.output = out.data_ptr()
        a.output_stride = out.stride(0) * out.element_size()
        a.output_dtype = capi.DTYPE_FLOAT16 if out.dtype == torch.float16 else capi.DTYPE_FLOAT32
        capi.check(capi.lib.nve_b200_lookup_pool(C.byref(a), self._stream()))

    def close(self):
        if self.deduper:
            capi.check(capi.lib.nve_b200_deduper_destroy(self.deduper))
            self.deduper = None


def allocate_symmetric_shard(rows: int, dim: int, dtype: torch.dtype) -> torch.Tensor:
    """Shard storage that every rank of the job can map (torch symmetric memory); required for
    ``mode="peer"``.  Fill it, then hand it to :class:`ShardedEmbeddingTable`."""
    import torch.distributed._symmetric_memory as symm_mem
    return symm_mem.empty((rows, dim), dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))


class ShardedEmbeddingTable:
    """A table of ``world * local_rows`` rows sharded round-robin over the ranks of a process group.

    mode="alltoall": dedup + two all-to-all exchanges (every distinct row crosses NVLink once).
    mode="peer":     every rank maps all shards (symmetric memory) and ONE fused kernel probes,
                     reads the rows straight from their owners over NVLink and pools them; no
                     collective, no host synchronisation on the lookup path.
    """

    POOLING = {"sum": capi.POOL_SUM, "mean": capi.POOL_MEAN}

    def __init__(self, local_shard: torch.Tensor, *, max_keys: int, group=None, stages=None,
                 mode: str = "alltoall", cache_bytes: int = 0, monitor: PeerMonitor | None = None):
        self.group = group
        self.monitor = monitor       # optional host-side membership check before every lookup
        self.failed = None           # the error that ended the exchange form, once one has
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.shard = local_shard
        self.mode = mode
        self.last_exchange = {}
        self.stages = None
        if mode == "peer":
            if self.world > 1:
                import torch.distributed._symmetric_memory as symm_mem
                handle = symm_mem.rendezvous(local_shard, group if group is not None else dist.group.WORLD)
                self._symm = handle
                ptrs = [int(p) for p in handle.buffer_ptrs]
                torch.cuda.synchronize()
                dist.barrier(group)          # every shard is filled before anyone reads it
            else:
                ptrs = [local_shard.data_ptr()]
            self._shard_ptrs = (C.c_void_p * len(ptrs))(*ptrs)
            self._cache = None
            self.use_cache = True          # set False to bypass the cache without dropping it
            if cache_bytes > 0:
                # a local set-associative cache in front of the peer reads (mode="peer" only): rows
                # it holds are served from this GPU's HBM, the others from their owner over NVLink
                from .layers import GpuTable
                row_bytes = local_shard.shape[1] * local_shard.element_size()
                dt = "float16" if local_shard.dtype == torch.float16 else "float32"
                self._cache = GpuTable(cache_bytes, row_bytes, dt, max_modify_size=max(max_keys, 1),
                                       device_id=local_shard.device.index)
                self._cache_ctx = self._cache.create_execution_context()
                self._cache_view = capi.CacheData()
                capi.check(capi.lib.nve_b200_gpu_table_get_cache_data(
                    self._cache.handle, self._cache_ctx.handle, C.byref(self._cache_view)))
        else:
            self.stages = stages if stages is not None else CudaStages(max_keys, self.world)

    def populate_cache(self, keys: torch.Tensor):
        """Insert the rows of `keys` (global row ids) into the local cache, most frequent first
        (the cache's replacement policy).  Call between lookups; returns after the insert ran."""
        if self._cache is None:
            raise RuntimeError("the table was created without a cache")
        n = keys.numel()
        rows = self._lookup_peer(keys, "sum", 1, None, None, use_cache=False)   # one row per key
        torch.cuda.current_stream().synchronize()
        row_bytes = self.shard.shape[1] * self.shard.element_size()
        self._cache.insert(self._cache_ctx, n, keys, row_bytes, row_bytes, rows)
        self._cache_ctx.wait()

    def cache_misses(self, reset: bool = False) -> int:
        """Keys not served by the local cache since the counter was last reset (synchronises)."""
        torch.cuda.current_stream().synchronize()
        v = C.c_int64(0)
        capi.check(capi.lib.nve_table_get_lookup_counter(self._cache.handle, self._cache_ctx.handle, C.byref(v)))
        self._cache_ctx.wait()
        if reset:
            capi.check(capi.lib.nve_table_reset_lookup_counter(self._cache.handle, self._cache_ctx.handle))
            self._cache_ctx.wait()
        return v.value

    def _lookup_peer(self, keys, pooling, fixed_hotness, csr_offsets, out, use_cache=True):
        n = keys.numel()
        num_bags = (csr_offsets.numel() - 1) if csr_offsets is not None else n // fixed_hotness
        if out is None:
            out = torch.empty((num_bags, self.shard.shape[1]), dtype=self.shard.dtype, device=keys.device)
        a = capi.PoolArgs()
        a.table = None
        a.num_rows = self.shard.shape[0] * self.world
        a.row_stride = self.shard.stride(0) * self.shard.element_size()
        a.value_dtype = capi.DTYPE_FLOAT16 if self.shard.dtype == torch.float16 else capi.DTYPE_FLOAT32
        a.row_width = self.shard.shape[1]
        a.default_row_index = -1
        cached = use_cache and self.use_cache and self._cache is not None
        a.cache = C.pointer(self._cache_view) if cached else None
        a.key_type = capi.KEY_INT64
        a.keys = keys.data_ptr()
        a.num_keys = n
        a.pooling_type = self.POOLING[pooling]
        a.sparse_type = capi.SPARSE_CSR if csr_offsets is not None else capi.SPARSE_FIXED
        a.csr_offsets = csr_offsets.data_ptr() if csr_offsets is not None else None
        a.offset_bytes = 8
        a.num_bags = num_bags
        a.fixed_hotness = fixed_hotness
        a.weights = None
        a.output = out.data_ptr()
        a.output_stride = out.stride(0) * out.element_size()
        a.output_dtype = capi.DTYPE_FLOAT16 if out.dtype == torch.float16 else capi.DTYPE_FLOAT32
        if self.world > 1:
            a.shard_tables = self._shard_ptrs
            a.num_shards = self.world
        else:                       # one rank: the shard is the table
            a.table = self.shard.data_ptr()
        capi.check(capi.lib.nve_b200_lookup_pool(C.byref(a), torch.cuda.current_stream().cuda_stream))
        row_bytes = self.shard.shape[1] * self.shard.element_size()
        self.last_exchange = {"unique": None, "served": None, "cached": bool(cached),
                              "nvlink_bytes_in": n * row_bytes * (self.world - 1) // self.world}
        return out

    def lookup_pooled(self, keys: torch.Tensor, pooling: str = "sum", *, fixed_hotness: int = 0,
                      csr_offsets: torch.Tensor | None = None, out: torch.Tensor | None = None):
        if self.monitor is not None:
            self.monitor.check()
        if self.mode == "peer":
            return self._lookup_peer(keys, pooling, fixed_hotness, csr_offsets, out)
        if self.failed is not None:
            raise ExchangeFailed(f"an earlier exchange failed: {self.failed}")
        try:
            return self._lookup_exchange(keys, pooling, fixed_hotness, csr_offsets, out)
        except (PeerLeft, ExchangeFailed, capi.NveError):
            raise
        except RuntimeError as e:        # torch.distributed reports dead peers and timeouts this way
            if self.world == 1:
                raise
            self.failed = str(e).splitlines()[0] if str(e) else type(e).__name__
            raise ExchangeFailed(f"exchange with the other ranks failed: {self.failed}") from e

    def _lookup_exchange(self, keys, pooling, fixed_hotness, csr_offsets, out):
        n = keys.numel()
        w = self.world
        send_keys, send_counts = self.stages.dedup_and_route(keys)
        if w > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
            # the one host read-back of a lookup: NCCL takes the split sizes from the host
            both = _split_list(torch.cat([send_counts, recv_counts]))
            send_splits, recv_splits = both[:w], both[w:]
            u = sum(send_splits)
            send_keys = send_keys[:u]
            recv_keys = torch.empty(sum(recv_splits), dtype=send_keys.dtype, device=send_keys.device)
            dist.all_to_all_single(recv_keys, send_keys.contiguous(), recv_splits, send_splits,
                                   group=self.group)
        else:
            u = _split_list(send_counts)[0]
            send_splits = recv_splits = [u]
            recv_keys = send_keys[:u].clone()
        served = self.stages.serve(self.shard, recv_keys)
        if w > 1:
            rows = torch.empty((u, self.shard.shape[1]), dtype=self.shard.dtype, device=served.device)
            dist.all_to_all_single(rows, served, send_splits, recv_splits, group=self.group)
        else:
            rows = served
        num_bags = (csr_offsets.numel() - 1) if csr_offsets is not None else n // fixed_hotness
        if out is None:
            out = torch.empty((num_bags, self.shard.shape[1]), dtype=self.shard.dtype, device=rows.device)
        self.stages.pool(rows, n, self.POOLING[pooling], fixed_hotness, csr_offsets, out)
        row_bytes = self.shard.shape[1] * self.shard.element_size()
        remote = u - send_splits[self.rank] if w > 1 else 0
        self.last_exchange = {"unique": u, "served": int(recv_keys.numel()),
                              "nvlink_bytes_out": remote * 8 + (int(recv_keys.numel()) - recv_splits[self.rank]) * row_bytes if w > 1 else 0}
        return out

    def close(self):
        if self.stages is not None and hasattr(self.stages, "close"):
            self.stages.close()
        if getattr(self, "_cache", None) is not None:
            self._cache_ctx.wait()
            self._cache_ctx.destroy()
            self._cache.destroy()
            self._cache = None
