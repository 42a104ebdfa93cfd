"""Row-sharded embedding table over several GPUs, one process per GPU.

Row ``r`` of the global table lives on rank ``r mod W`` at local index ``r // W``.  The table is the
C++ object ``nve_b200_sharded_table_*`` of libnve_b200; this module is its ctypes veneer plus the
set-up that needs the job's process group (exchanging shard addresses or the NCCL id).  Nothing of
torch.distributed is on the lookup path.

``mode="peer"`` (the one to use on NVLink): every rank allocates its shard in symmetric memory, the
ranks exchange the mapped base addresses once, and ONE fused kernel reads each row from its owner's
HBM and pools — no collective and no host synchronisation per lookup.  This is what the reference
does with one address range mapped over all shards (src/distributed.cpp:155-256,
src/memblock_nvl.cpp:40-119).  ``hot_rows`` puts a replicated hot-row table in front: the rows a
sample of the key stream asks for most (:meth:`set_hot_keys`) are copied into every GPU's own HBM
and never cross NVLink again.  ``cache_bytes`` (instead) puts the set-associative cache in front.

``mode="alltoall"``: every lookup de-duplicates its keys, sends each distinct key once to its owner,
the owners read their rows, the rows come back, and the batch is pooled from the received rows.  The
exchanges are ncclSend / ncclRecv groups issued by the library on a communicator of its own; one
host wait per lookup (the per-owner key counts).  ``hot_rows`` works here too: hot keys take no part
in the exchange.

Results of every form are those of a lookup in the unsharded table.

``stages`` replaces the device stages by a host implementation and runs the exchange protocol in
Python over ``torch.distributed`` (any backend): that is how the rank logic (split sizes, ordering,
failure reporting) is tested with CPU ranks.
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


def _dtype_id(t: torch.dtype) -> int:
    if t == torch.float16:
        return capi.DTYPE_FLOAT16
    if t == torch.float32:
        return capi.DTYPE_FLOAT32
    raise TypeError(f"sharded table: rows must be float16 or float32, not {t}")


class ShardedEmbeddingTable:
    """A table of ``world * local_rows`` rows sharded round-robin over the ranks of a process group.

    mode="peer":     every rank maps all shards (symmetric memory) and ONE fused kernel reads the
                     rows from their owners over NVLink and pools them; no collective, no host
                     synchronisation on the lookup path.
    mode="alltoall": hash dedup + two ncclSend/ncclRecv exchanges inside libnve_b200 (every distinct
                     row crosses NVLink once).  Collective: every rank calls lookup_pooled.
    hot_rows > 0:    a replicated table of that many rows in front of either form (set_hot_keys).
    cache_bytes > 0: (peer only, instead of hot_rows) the set-associative cache in front.
    transport:       (alltoall) a capi.ExchangeOps of the caller's instead of the built-in NCCL one.
    stages:          run the exchange protocol in Python with these stage implementations (tests).
    """

    POOLING = {"sum": capi.POOL_SUM, "mean": capi.POOL_MEAN, "weighted_sum": capi.POOL_WEIGHTED_SUM,
               "weighted_mean": capi.POOL_WEIGHTED_MEAN}

    def __init__(self, local_shard: torch.Tensor, *, max_keys: int, group=None, stages=None,
                 mode: str = "alltoall", cache_bytes: int = 0, hot_rows: int = 0,
                 monitor: PeerMonitor | None = None, transport=None, world: int | None = None,
                 rank: int | None = None, peer_shards=None, default_row: int = -1,
                 timeout_ms: int = 0):
        self.group = group
        self.monitor = monitor       # optional host-side membership check before every lookup
        self.failed = None           # the error that ended the exchange form, once one has
        if world is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world, self.rank = world, rank
        self.shard = local_shard
        self.mode = mode
        self.max_keys = max_keys
        self.last_exchange = {}
        self.stages = stages
        self.handle = None
        self._cache = None
        self.use_cache = True          # set False to bypass the cache without dropping it
        if mode not in ("peer", "alltoall"):
            raise ValueError(f"unknown mode {mode!r}")
        if stages is not None:
            if mode != "alltoall":
                raise ValueError("stages run the exchange form")
            return
        ptrs = None
        if mode == "peer":
            if peer_shards is not None:
                ptrs = [int(p) for p in peer_shards]
            elif self.world > 1:
                import torch.distributed._symmetric_memory as symm_mem
                handle = symm_mem.rendezvous(local_shard, group if group is not None else dist.group.WORLD)
                self._symm = handle
                ptrs = [int(p) for p in handle.buffer_ptrs]
                torch.cuda.synchronize()
                dist.barrier(group)          # every shard is filled before anyone reads it
            else:
                ptrs = [local_shard.data_ptr()]
            self._shard_ptrs = (C.c_void_p * len(ptrs))(*ptrs)
            if cache_bytes > 0:
                # a local set-associative cache in front of the peer reads: rows it holds are served
                # from this GPU's HBM, the others from their owner over NVLink (general kernel)
                if hot_rows > 0:
                    raise ValueError("cache_bytes and hot_rows are alternatives")
                from .layers import GpuTable
                row_bytes = local_shard.shape[1] * local_shard.element_size()
                dt = "float16" if local_shard.dtype == torch.float16 else "float32"
                self._cache = GpuTable(cache_bytes, row_bytes, dt, max_modify_size=max(max_keys, 1),
                                       device_id=local_shard.device.index)
                self._cache_ctx = self._cache.create_execution_context()
                self._cache_view = capi.CacheData()
                capi.check(capi.lib.nve_b200_gpu_table_get_cache_data(
                    self._cache.handle, self._cache_ctx.handle, C.byref(self._cache_view)))
        cfg = capi.ShardedTableConfig()
        cfg.world, cfg.rank = self.world, self.rank
        cfg.device_id = local_shard.device.index if local_shard.device.index is not None else torch.cuda.current_device()
        cfg.mode = capi.SHARD_PEER if mode == "peer" else capi.SHARD_EXCHANGE
        cfg.local_shard = local_shard.data_ptr()
        cfg.local_rows = local_shard.shape[0]
        cfg.row_stride = local_shard.stride(0) * local_shard.element_size()
        cfg.value_dtype = _dtype_id(local_shard.dtype)
        cfg.row_width = local_shard.shape[1]
        cfg.key_type = capi.KEY_INT64
        cfg.default_row_index = default_row
        cfg.max_keys = max_keys
        cfg.hot_capacity = hot_rows
        cfg.exchange_timeout_ms = timeout_ms
        if ptrs is not None:
            cfg.peer_shards = self._shard_ptrs
        self._transport = transport       # keeps the callbacks alive
        if mode == "alltoall" and self.world > 1:
            if transport is not None:
                cfg.exchange_ops = C.pointer(transport)
            else:
                uid = (C.c_char * 128)()
                if self.rank == 0:
                    capi.check(capi.lib.nve_b200_nccl_unique_id(uid))
                box = [bytes(uid)]
                dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0,
                                           group=group)
                self._uid = C.create_string_buffer(box[0], 128)
                cfg.nccl_unique_id = C.cast(self._uid, C.c_void_p)
        h = C.c_void_p()
        capi.check(capi.lib.nve_b200_sharded_table_create(C.byref(h), C.byref(cfg)))   # collective (NCCL id)
        self.handle = h
        self.hot_rows = 0

    # ---- hot rows ------------------------------------------------------------------------------
    def set_hot_keys(self, keys: torch.Tensor) -> int:
        """Chooses the hot rows from a sample of the key stream (repeats count) and copies them into
        this GPU's memory; returns how many rows are hot.  Call between lookups; collective in the
        exchange form."""
        n = C.c_int64(0)
        capi.check(capi.lib.nve_b200_sharded_table_set_hot_keys(
            self.handle, keys.data_ptr() if keys.numel() else None, keys.numel(), C.byref(n),
            torch.cuda.current_stream().cuda_stream))
        self.hot_rows = n.value
        return n.value

    # ---- the set-associative cache in front of the peer reads (general kernel) -------------------
    def populate_cache(self, keys: torch.Tensor):
        """Insert the rows of `keys` (global row ids) into the local cache, most frequent first
        (the cache's replacement policy).  Call between lookups; returns after the insert ran."""
        if self._cache is None:
            raise RuntimeError("the table was created without a cache")
        n = keys.numel()
        rows = self._lookup_cached(keys, "sum", 1, None, None, use_cache=False)   # one row per key
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

    def _lookup_cached(self, keys, pooling, fixed_hotness, csr_offsets, out, use_cache=True):
        n = keys.numel()
        num_bags = (csr_offsets.numel() - 1) if csr_offsets is not None else n // fixed_hotness
        if out is None:
            out = torch.empty((num_bags, self.shard.shape[1]), dtype=self.shard.dtype, device=keys.device)
        a = capi.PoolArgs()
        a.table = None
        a.num_rows = self.shard.shape[0] * self.world
        a.row_stride = self.shard.stride(0) * self.shard.element_size()
        a.value_dtype = _dtype_id(self.shard.dtype)
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
        a.output_dtype = _dtype_id(out.dtype)
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

    # ---- lookups -------------------------------------------------------------------------------
    def lookup_pooled(self, keys: torch.Tensor, pooling: str = "sum", *, fixed_hotness: int = 0,
                      csr_offsets: torch.Tensor | None = None, out: torch.Tensor | None = None,
                      weights: torch.Tensor | None = None):
        if self.monitor is not None:
            self.monitor.check()
        if self.stages is not None:
            if self.failed is not None:
                raise ExchangeFailed(f"an earlier exchange failed: {self.failed}")
            try:
                return self._lookup_protocol(keys, pooling, fixed_hotness, csr_offsets, out)
            except (PeerLeft, ExchangeFailed, capi.NveError):
                raise
            except RuntimeError as e:        # torch.distributed reports dead peers and timeouts this way
                if self.world == 1:
                    raise
                self.failed = str(e).splitlines()[0] if str(e) else type(e).__name__
                raise ExchangeFailed(f"exchange with the other ranks failed: {self.failed}") from e
        if self._cache is not None and self.use_cache:
            return self._lookup_cached(keys, pooling, fixed_hotness, csr_offsets, out)
        if self.failed is not None:
            raise ExchangeFailed(f"an earlier exchange failed: {self.failed}")
        n = keys.numel()
        num_bags = (csr_offsets.numel() - 1) if csr_offsets is not None else n // fixed_hotness
        if out is None:
            out = torch.empty((num_bags, self.shard.shape[1]), dtype=self.shard.dtype, device=keys.device)
        a = capi.ShardedLookup()
        a.keys = keys.data_ptr() if n else None
        a.num_keys = n
        a.pooling_type = self.POOLING[pooling]
        a.sparse_type = capi.SPARSE_CSR if csr_offsets is not None else capi.SPARSE_FIXED
        a.csr_offsets = csr_offsets.data_ptr() if csr_offsets is not None else None
        a.offset_bytes = csr_offsets.element_size() if csr_offsets is not None else 8
        a.num_bags = num_bags
        a.fixed_hotness = fixed_hotness
        if weights is not None:
            a.weights = weights.data_ptr()
            a.weight_dtype = _dtype_id(weights.dtype)
        a.output = out.data_ptr()
        a.output_stride = out.stride(0) * out.element_size()
        a.output_dtype = _dtype_id(out.dtype)
        st = capi.lib.nve_b200_sharded_table_lookup_pooled(self.handle, C.byref(a),
                                                           torch.cuda.current_stream().cuda_stream)
        if st == capi.NVE_ERROR_RUNTIME and self.mode == "alltoall" and self.world > 1:
            self.failed = capi.last_error()
            raise ExchangeFailed(f"exchange with the other ranks failed: {self.failed}")
        capi.check(st)
        row_bytes = self.shard.shape[1] * self.shard.element_size()
        if self.mode == "peer":
            self.last_exchange = {"unique": None, "served": None, "hot_rows": self.hot_rows,
                                  "nvlink_bytes_in": None if self.hot_rows else
                                  n * row_bytes * (self.world - 1) // self.world}
        else:
            stats = (C.c_int64 * 8)()
            capi.check(capi.lib.nve_b200_sharded_table_stats(self.handle, stats))
            self.last_exchange = {"unique": stats[0] if stats[0] >= 0 else None,
                                  "served": stats[1] if stats[1] >= 0 else None,
                                  "hot_rows": int(stats[2]), "nvlink_bytes_out": int(stats[3])}
        return out

    def _lookup_protocol(self, keys, pooling, fixed_hotness, csr_offsets, out):
        """The exchange protocol in Python over torch.distributed, with `self.stages` doing the
        device (or, in tests, host) stages."""
        n = keys.numel()
        w = self.world
        send_keys, send_counts = self.stages.dedup_and_route(keys)
        if w > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
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
        if self.handle is not None:
            capi.check(capi.lib.nve_b200_sharded_table_destroy(self.handle))
            self.handle = None
        if getattr(self, "_cache", None) is not None:
            self._cache_ctx.wait()
            self._cache_ctx.destroy()
            self._cache.destroy()
            self._cache = None
