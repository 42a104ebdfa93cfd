"""Benchmark drivers for the other configurations of the lookup hot path (bench.py runs the
headline one).  Each function builds seeded synthetic inputs of the configuration's shape on the
current CUDA device, times the path with CUDA events and returns a dict (one JSON line).

    python bench.py --workload c3|c4a|c4b|c5 [--steps K] [--warmup W]
"""
from __future__ import annotations

import ctypes as C
import json
import os
import time

import numpy as np
import torch

from . import capi, datagen as dg
from .layers import GpuTable, GPUEmbeddingLayer, LinearUVMEmbeddingLayer


def _hbm_peak(root):
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _time_loop(stream, fn, steps, warmup):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        fn(warmup + i)
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / steps


def _fill_rows_fp16(dst: torch.Tensor, seed: int, std: float = 0.02, chunk: int = 1 << 22):
    """dst: [rows, dim] fp16 tensor (device or pinned host), filled chunk-wise from a device RNG."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    for r0 in range(0, dst.shape[0], chunk):
        r1 = min(dst.shape[0], r0 + chunk)
        dst[r0:r1].copy_((torch.randn((r1 - r0, dst.shape[1]), generator=gen, device="cuda") * std).half())


def h2d_probe_gbs(nbytes: int = 1 << 30, reps: int = 10) -> float:
    """Host-link ceiling: pinned host -> device copy, best of `reps`."""
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    best = 1e9
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        d.copy_(h, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e-3)
    return nbytes / best / 1e9


def run_c3(root, steps=50, warmup=5, rows=100_000_000, dim=128, batch=262_144, cache_frac=0.10, ref_gpu=None):
    """LinearUVM cached lookup, no pooling: table in host memory (a managed block advised to the
    host, or cudaHostAlloc'ed memory with NVE_B200_C3_TABLE=pinned), 10 % of rows cached."""
    row_bytes = dim * 2
    stream = torch.cuda.current_stream()
    # Table storage: a managed block advised to stay in host memory (what the reference's
    # ManagedMemBlock gives a LinearUVM layer).  NVE_B200_C3_TABLE=pinned uses cudaHostAlloc'ed
    # memory instead, for the comparison quoted in the design notes.
    storage = os.environ.get("NVE_B200_C3_TABLE", "managed")
    if storage == "managed":
        from .memblock import ManagedMemBlock
        block = ManagedMemBlock(rows * row_bytes, (torch.cuda.current_device(),))
        table = block.as_tensor((rows, dim), torch.float16)
    else:
        block = None
        table = torch.empty((rows, dim), dtype=torch.float16).pin_memory()
    _fill_rows_fp16(table, 30)
    cache_bytes = int(rows * cache_frac) * row_bytes
    gt = GpuTable(cache_bytes, row_bytes, "float16", uvm_table=table, uvm_num_rows=rows)
    layer = LinearUVMEmbeddingLayer(gt)
    ctx = layer.create_execution_context(stream.cuda_stream, stream.cuda_stream)
    import time
    insert_s = []
    for b in range(20):                                    # explicit, deterministic warm-up
        k = torch.from_numpy(dg.zipf_keys(batch, rows, 1.2, 300 + b)).cuda()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        capi.check(capi.lib.nve_b200_gpu_table_insert_from_backing(gt.handle, ctx.handle, batch, k.data_ptr()))
        ctx.wait()
        insert_s.append(time.perf_counter() - t0)
    out = torch.empty((batch, dim), dtype=torch.float16, device="cuda")
    link = h2d_probe_gbs()
    peak, kind = _hbm_peak(root)
    res = {"workload": "C3 LinearUVM: 100M x 128 fp16 in host memory, 10% GPU cache, 262144 keys, no pooling",
           "host_link_probe_gbs": link, "table_storage": storage,
           "insert_us_median": float(np.median(insert_s[5:]) * 1e6), "gather": "bulk-copy" if os.environ.get("NVE_B200_GATHER_BULK") == "1" else "lane-vector",
           "runs": {}}
    nb = 16   # distinct batches per run, cycled: missed rows must come over the link every time
    for name, gen_keys in (("zipf1.2", lambda b: dg.zipf_keys(batch, rows, 1.2, 320 + 2 * b)),
                           ("uniform", lambda b: dg.uniform_keys(batch, rows, 321 + 2 * b))):
        keys_np = gen_keys(0)
        batches = [torch.from_numpy(gen_keys(b)).cuda() for b in range(nb)]
        hr = layer.lookup(ctx, batch, batches[0], out, row_bytes, want_hitrate=True)
        ctx.wait()
        ok = bool(torch.equal(out.cpu(), table[torch.from_numpy(keys_np)]))
        hrs = [layer.lookup(ctx, batch, k, out, row_bytes, want_hitrate=True) for k in batches]
        hr = float(np.mean(hrs))
        sec = _time_loop(stream, lambda i: layer.lookup(ctx, batch, batches[i % nb], out, row_bytes),
                         steps, warmup)
        misses = round((1.0 - hr) * batch)
        res["runs"][name] = {
            "keys_per_s": batch / sec, "us_per_lookup": sec * 1e6, "hit_rate": hr, "byte_exact": ok,
            "algorithmic_gbs": batch * (8 + 2 * row_bytes) / sec / 1e9,
            "hbm_gbs": ((batch - misses) * 2 * row_bytes + misses * row_bytes + batch * 8) / sec / 1e9,
            "host_link_gbs": misses * row_bytes / sec / 1e9,
            "host_link_frac_of_probe": misses * row_bytes / sec / 1e9 / link,
            "frac_of_hbm_peak": batch * (8 + 2 * row_bytes) / sec / 1e9 / peak, "peak_kind": kind}
    res["schedules"] = _c3_schedules(gt, ctx, table, rows, row_bytes, batch, stream, steps, warmup)
    ctx.destroy(); layer.destroy(); gt.destroy()
    # the pipeline schedule (host threads gather the missed rows): its own table, warmed the same way
    gt = GpuTable(cache_bytes, row_bytes, "float16", uvm_table=table, uvm_num_rows=rows, kernel_mode_type=3)
    ctx = gt.create_execution_context(stream.cuda_stream, stream.cuda_stream)
    for b in range(20):
        k = torch.from_numpy(dg.zipf_keys(batch, rows, 1.2, 300 + b)).cuda()
        capi.check(capi.lib.nve_b200_gpu_table_insert_from_backing(gt.handle, ctx.handle, batch, k.data_ptr()))
    ctx.wait()
    res["pipeline_schedule"] = {}
    for name, gen_keys in (("zipf1.2", lambda b: dg.zipf_keys(batch, rows, 1.2, 320 + 2 * b)),
                           ("uniform", lambda b: dg.uniform_keys(batch, rows, 321 + 2 * b))):
        keys_np = gen_keys(0)
        batches = [torch.from_numpy(gen_keys(b)).cuda() for b in range(4)]
        gt.find(ctx, batch, batches[0], None, row_bytes, out)
        ctx.wait()
        ok = bool(torch.equal(out.cpu(), table[torch.from_numpy(keys_np)]))
        sec = _time_loop(stream, lambda i: gt.find(ctx, batch, batches[i % 4], None, row_bytes, out),
                         min(steps, 20), 3)
        res["pipeline_schedule"][name] = {"us_per_lookup": sec * 1e6, "byte_exact": ok}
    ctx.destroy(); gt.destroy()
    if ref_gpu is not None:
        # the reference cache, warmed with the same insert sequence, serving the same batches
        rc = ref_gpu.cache(cache_bytes, row_bytes, max_modify=batch)
        ref_insert_s = []
        for b in range(20):
            k = torch.from_numpy(dg.zipf_keys(batch, rows, 1.2, 300 + b)).cuda()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            rc.insert_from_table(k.data_ptr(), batch, table.data_ptr(), row_bytes)
            ref_insert_s.append(time.perf_counter() - t0)
        res["reference_gpu"] = {"insert_us_median": float(np.median(ref_insert_s[5:]) * 1e6)}
        for name, gen_keys in (("zipf1.2", lambda b: dg.zipf_keys(batch, rows, 1.2, 320 + 2 * b)),
                               ("uniform", lambda b: dg.uniform_keys(batch, rows, 321 + 2 * b))):
            batches = [torch.from_numpy(gen_keys(b)).cuda() for b in range(nb)]
            misses = rc.lookup_table(batches[0].data_ptr(), batch, out.data_ptr(), row_bytes, table.data_ptr())
            ms = rc.lookup_table_timed([k.data_ptr() for k in batches], batch, out.data_ptr(), row_bytes,
                                       table.data_ptr(), warmup, steps)
            res["reference_gpu"][name] = {"us_per_lookup": ms * 1e3, "keys_per_s": batch / (ms * 1e-3),
                                          "hit_rate_first_batch": 1.0 - misses / batch}
        rc.close()
    del table
    if block is not None:
        block.close()
    return res


def run_published_gpulayer(root, steps=50, warmup=5, rows=250_000_000, dim=128, batch=262_144):
    """The shape of the reference's own published GPULayer benchmark (docs/benchmarks.md: fp32, dim 128,
    128 GB table in HBM, 256 x 1024 keys per step, power-law keys alpha 1.05, un-pooled lookups,
    device-resident keys): one un-pooled lookup of `batch` keys per step through the dense layer."""
    stream = torch.cuda.current_stream()
    row_bytes = dim * 4
    table = torch.empty((rows, dim), dtype=torch.float32, device="cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(70)
    chunk = 1 << 22
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        table[r0:r1].normal_(0, 0.02, generator=gen)
    layer = GPUEmbeddingLayer(table, rows, row_bytes, "float32")
    ctx = layer.create_execution_context(stream.cuda_stream, stream.cuda_stream)
    nb = 8
    # power-law ranks spread over the table by a multiplicative bijection of Z_rows (the multiplier is a
    # prime that does not divide `rows`), standing in for the reference's random permutation, which
    # at this size would take gigabytes of host memory to build
    def spread(ranks):
        return ((ranks.astype(np.uint64) * np.uint64(2654435761)) % np.uint64(rows)).astype(np.int64)
    batches = [torch.from_numpy(spread(dg.zipf_keys(batch, rows, 1.05, 700 + b))).cuda() for b in range(nb)]
    out = torch.empty((batch, dim), dtype=torch.float32, device="cuda")
    layer.lookup(ctx, batch, batches[0], out, row_bytes)
    ctx.wait()
    ok = bool(torch.equal(out, table[batches[0]]))
    sec = _time_loop(stream, lambda i: layer.lookup(ctx, batch, batches[i % nb], out, row_bytes), steps, warmup)
    peak, kind = _hbm_peak(root)
    alg = batch * (8 + 2 * row_bytes)
    res = {"workload": f"published GPULayer shape: {rows} x {dim} fp32 in HBM ({rows * row_bytes / 1e9:.0f} GB), "
                       f"{batch} keys per step, power-law 1.05, un-pooled",
           "keys_per_s": batch / sec, "mkps": batch / sec / 1e6, "us_per_lookup": sec * 1e6,
           "algo_bw_gib_s": batch / sec * row_bytes / 2**30, "algorithmic_gbs": alg / sec / 1e9,
           "frac_of_hbm_peak": alg / sec / 1e9 / peak, "peak_kind": kind, "byte_exact": ok,
           "reference_published": {"mkps": 2910.36, "algo_bw_gib_s": 1387.77, "hardware": "1x GB200",
                                   "source": "docs/benchmarks.md:40-42"}}
    ctx.destroy()
    layer.destroy()
    return res


def _c3_schedules(gt, ctx, table, rows, row_bytes, batch, stream, steps, warmup):
    """The fused lookup kernel and the sort-gather schedule through the kernel-level C ABI on the warmed
    cache of the C3 run: the configuration's batch and one eight times larger, Zipf and uniform keys."""
    view = capi.CacheData()
    capi.check(capi.lib.nve_b200_gpu_table_get_cache_data(gt.handle, ctx.handle, C.byref(view)))
    out = {}
    nb = 4
    for n in (batch, 8 * batch):
        rows_out = torch.empty((n, row_bytes), dtype=torch.uint8, device="cuda")
        for name, gen_keys in (("zipf1.2", lambda b: dg.zipf_keys(n, rows, 1.2, 340 + 2 * b)),
                               ("uniform", lambda b: dg.uniform_keys(n, rows, 341 + 2 * b))):
            batches = [torch.from_numpy(gen_keys(b)).cuda() for b in range(nb)]
            g = capi.GatherArgs()
            g.table, g.num_rows, g.row_stride = table.data_ptr(), rows, row_bytes
            g.value_dtype = g.output_dtype = capi.DTYPE_FLOAT16
            g.default_row_index, g.cache, g.key_type = -1, C.pointer(view), capi.KEY_INT64
            g.num_keys, g.output, g.output_stride, g.row_copy_bytes = n, rows_out.data_ptr(), row_bytes, row_bytes
            need = C.c_size_t(0)
            g.keys = batches[0].data_ptr()
            capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), 0, None, C.byref(need), None))
            scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")
            s = stream.cuda_stream

            def fused(i):
                g.keys = batches[i % nb].data_ptr()
                capi.check(capi.lib.nve_b200_gather_rows(C.byref(g), s))

            def ordered(i):
                g.keys = batches[i % nb].data_ptr()
                capi.check(capi.lib.nve_b200_gather_rows_sorted(C.byref(g), 0, scratch.data_ptr(), C.byref(need), s))
            ordered(0)
            stream.synchronize()
            first = rows_out.clone()
            fused(0)
            stream.synchronize()
            identical = bool(torch.equal(first, rows_out))
            out[f"{name}_{n}"] = {"us_fused": _time_loop(stream, fused, steps, warmup) * 1e6,
                                  "us_sort_gather": _time_loop(stream, ordered, steps, warmup) * 1e6,
                                  "identical": identical}
            del scratch
        del rows_out
    return out


def _quant_table(rows, width, stride, seed):
    t = torch.zeros((rows, stride), dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    chunk = 1 << 21
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        t[r0:r1, :width] = torch.randint(-127, 128, (r1 - r0, width), generator=gen, device="cuda",
                                         dtype=torch.int8).view(torch.uint8)
        scale = torch.rand((r1 - r0, 1), generator=gen, device="cuda") * 9e-3 + 1e-3
        t[r0:r1, width:width + 4] = scale.view(torch.uint8)
    return t


def run_c4a(root, steps=50, warmup=5, rows=50_000_000, width=256, bags=32_768, hot=20, ref_gpu=None):
    """find_and_dequant + sum pooling: int8 rows with fp32 row scale -> fp16 sums.  Four key batches
    are cycled.  `ref_gpu`: optional handle of the reference GPU code, timed beside on the tight
    layout (it writes fp32 sums: the reference has no fp16 output for fp32-scaled rows)."""
    stream = torch.cuda.current_stream()
    peak, kind = _hbm_peak(root)
    batches = [torch.from_numpy(dg.zipf_keys(bags * hot, rows, 1.05, 400 + b)).cuda() for b in range(4)]
    keys = batches[0]
    out = torch.empty((bags, width), dtype=torch.float16, device="cuda")
    res = {"workload": "C4a: 50M x 256 int8 + fp32 scale, 32768 bags x 20 keys Zipf(1.05), dequant + sum -> fp16", "runs": {}}
    for stride in (width + 4, 272):
        t = _quant_table(rows, width, stride, 40)
        a = capi.PoolArgs()
        a.table, a.num_rows, a.row_stride = t.data_ptr(), rows, stride
        a.value_dtype, a.row_width, a.default_row_index = capi.DTYPE_QINT8_F32, width, -1
        a.cache, a.key_type, a.keys, a.num_keys = None, capi.KEY_INT64, keys.data_ptr(), keys.numel()
        a.pooling_type, a.sparse_type, a.num_bags, a.fixed_hotness = capi.POOL_SUM, capi.SPARSE_FIXED, bags, hot
        a.output, a.output_stride, a.output_dtype = out.data_ptr(), width * 2, capi.DTYPE_FLOAT16

        def launch(i):
            a.keys = batches[i % 4].data_ptr()
            capi.check(capi.lib.nve_b200_lookup_pool(C.byref(a), stream.cuda_stream))
        sec = _time_loop(stream, launch, steps, warmup)
        alg = keys.numel() * (8 + width + 4) + bags * width * 2
        res["runs"][f"stride{stride}"] = {"keys_per_s": keys.numel() / sec, "us_per_launch": sec * 1e6,
                                          "algorithmic_gbs": alg / sec / 1e9,
                                          "frac_of_hbm_peak": alg / sec / 1e9 / peak, "peak_kind": kind}
        if ref_gpu is not None and stride == width + 4:
            out32 = torch.empty((bags, width), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            ms = ref_gpu.find_and_combine("qint8_fixed_sum", bags, t.data_ptr(), [b.data_ptr() for b in batches],
                                          None, hot, width, out32.data_ptr(), warmup=warmup, iters=steps)
            res["reference_gpu_kernel"] = {"kernel": "find_and_combine (int8 + fp32 scale, fixed hotness, sum, fp32 out)",
                                           "layout": f"stride{stride}", "us_per_launch": ms * 1e3,
                                           "keys_per_s": keys.numel() / (ms * 1e-3)}
            del out32
        del t
        torch.cuda.empty_cache()
    return res


def run_c4b(root, steps=30, warmup=5, rows=10_000_000, dim=128, n=1_048_576, lr=0.01, ref_gpu=None):
    """dedup_grads + update_accumulate: 1M (key, grad) pairs into a 10M x 128 fp32 table."""
    stream = torch.cuda.current_stream()
    peak, kind = _hbm_peak(root)
    table = torch.empty((rows, dim), dtype=torch.float32, device="cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(50)
    table.normal_(0, 0.02, generator=gen)
    keys_np = dg.zipf_keys(n, rows, 1.05, 500)
    keys = torch.from_numpy(keys_np).cuda()
    grads = torch.empty((n, dim), dtype=torch.float32, device="cuda").normal_(0, 1e-2, generator=gen)
    i64 = dict(dtype=torch.int64, device="cuda")
    cap = n + n // 1024 + 2
    uniq, counts, inverse = torch.empty(n + 1, **i64), torch.empty(n + 1, **i64), torch.empty(n + 1, **i64)
    offsets, loc = torch.empty(cap + 1, **i64), torch.empty(cap + 1, **i64)
    d = C.c_void_p()
    capi.check(capi.lib.nve_b200_deduper_create(C.byref(d), capi.KEY_INT64, 1024, n))
    runs = (C.c_int64 * 2)()
    s = stream.cuda_stream

    def dedup(i):
        capi.check(capi.lib.nve_b200_deduper_dedup(d, keys.data_ptr(), n, uniq.data_ptr(), counts.data_ptr(),
                                                   loc.data_ptr(), runs, inverse.data_ptr(), offsets.data_ptr(), s, 24))

    def apply(i):
        capi.check(capi.lib.nve_b200_dedup_grads(d, grads.data_ptr(), dim * 4, dim * 4, n, uniq.data_ptr(),
                                                 inverse.data_ptr(), offsets.data_ptr(), loc.data_ptr(),
                                                 table.data_ptr(), dim * 4, 1, rows, -lr, s))
    t_dedup = _time_loop(stream, dedup, steps, warmup)
    u = int(runs[0])
    t_apply = _time_loop(stream, apply, steps, warmup)
    t_both = _time_loop(stream, lambda i: (dedup(i), apply(i)), steps, warmup)
    alg = n * (8 + dim * 4) + u * 2 * dim * 4
    capi.check(capi.lib.nve_b200_deduper_destroy(d))
    res = {"workload": "C4b: dedup_grads + update_accumulate, 1048576 pairs Zipf(1.05), 10M x 128 fp32, SGD lr 0.01",
           "unique": u, "keys_per_s": n / t_both, "us_dedup": t_dedup * 1e6, "us_reduce_apply": t_apply * 1e6,
           "us_total": t_both * 1e6, "algorithmic_gbs": alg / t_both / 1e9,
           "reduce_apply_gbs": alg / t_apply / 1e9, "frac_of_hbm_peak": alg / t_both / 1e9 / peak,
           "peak_kind": kind}
    if ref_gpu is not None:
        # the reference's three kernels for the same work: Deduper (sorting the same 24 key bits),
        # GradientDedup into a [unique, dim] buffer, UpdateAccumulateTable of that buffer into the table
        import time
        rd = ref_gpu.deduper(1024, n)
        ptrs = (keys.data_ptr(), n, uniq.data_ptr(), counts.data_ptr(), loc.data_ptr(), inverse.data_ptr(),
                offsets.data_ptr(), 24)
        for _ in range(warmup):
            ru, rc = rd.dedup(*ptrs)
        t0 = time.perf_counter()
        for _ in range(steps):
            ru, rc = rd.dedup(*ptrs)
        ref_dedup = (time.perf_counter() - t0) / steps
        sums = torch.empty((ru, dim), dtype=torch.float32, device="cuda")
        ms = rd.grads(grads.data_ptr(), sums.data_ptr(), uniq.data_ptr(), inverse.data_ptr(), loc.data_ptr(),
                      offsets.data_ptr(), ru, rc, dim, warmup=warmup, iters=steps)
        rd.close()
        ms_upd = ref_gpu.update_accumulate_table(sums.data_ptr(), uniq.data_ptr(), table.data_ptr(), dim, ru, rows,
                                                 warmup=warmup, iters=steps)
        res["reference_gpu"] = {"us_dedup": ref_dedup * 1e6, "us_reduce_only": ms * 1e3,
                                "us_update_accumulate": ms_upd * 1e3,
                                "us_total": ref_dedup * 1e6 + ms * 1e3 + ms_upd * 1e3,
                                "note": "reference Deduper (host-timed, includes its stream sync), GradientDedup "
                                        "and UpdateAccumulateTable of the summed rows (the scaling by the "
                                        "learning rate, a further pass there, is not included)"}
    return res


def run_c5(root, steps=30, warmup=5, rows_per_rank=250_000_000, dim=64, bags=131_072, hot=8,
           mode=os.environ.get("NVE_B200_SHARD_MODE", "peer")):
    """Row-sharded table, weak scaling: 32 GB of fp16 rows per rank, read over peer mappings
    (default) or served by dedup + all-to-all (NVE_B200_SHARD_MODE=alltoall)."""
    import torch.distributed as dist
    from .sharded import ShardedEmbeddingTable, allocate_symmetric_shard
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    stream = torch.cuda.current_stream()
    if mode == "peer" and world > 1:
        shard = allocate_symmetric_shard(rows_per_rank, dim, torch.float16)
    else:
        shard = torch.empty((rows_per_rank, dim), dtype=torch.float16, device="cuda")
    _fill_rows_fp16(shard, 60 + rank)
    total = rows_per_rank * world
    n = bags * hot
    # peer mode, optionally with a local cache in front of the peer reads: NVE_B200_C5_CACHE_FRAC is the
    # cache size as a fraction of the local shard's bytes (0 = no cache; the cached run is reported
    # beside the uncached one)
    cache_frac = float(os.environ.get("NVE_B200_C5_CACHE_FRAC", "0")) if mode == "peer" else 0.0
    row_bytes = dim * 2
    t = ShardedEmbeddingTable(shard, max_keys=n, mode=mode,
                              cache_bytes=int(rows_per_rank * cache_frac) * row_bytes)
    batches = [torch.from_numpy(dg.zipf_keys(n, total, 1.05, 600 + 10 * b + rank)).cuda() for b in range(4)]
    out = torch.empty((bags, dim), dtype=torch.float16, device="cuda")

    def step(i):
        t.lookup_pooled(batches[i % 4], "sum", fixed_hotness=hot, out=out)

    def timed():
        for i in range(warmup):
            step(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            step(warmup + i)
        e1.record(stream)
        torch.cuda.synchronize()
        sec = torch.tensor([e0.elapsed_time(e1) * 1e-3 / steps], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(sec, op=dist.ReduceOp.MAX)
        return float(sec.item())

    if cache_frac > 0:
        t.use_cache = False
    sec = timed()
    ex = dict(t.last_exchange)
    res = {"workload": "C5 sharded table: 250M x W rows x 64 fp16, 131072 bags x 8 per rank, Zipf(1.05), sum",
           "mode": mode, "n_gpus": world, "keys_per_s": n * world / sec, "ms_per_step": sec * 1e3,
           "unique_per_rank": ex.get("unique"), "served_per_rank": ex.get("served"),
           "nvlink_gbs_per_rank": (ex.get("nvlink_bytes_out") or ex.get("nvlink_bytes_in") or 0) / sec / 1e9,
           "scaling": "weak"}
    if cache_frac > 0:
        for b in range(12):                                   # explicit, deterministic warm-up of the cache
            k = torch.from_numpy(dg.zipf_keys(n, total, 1.05, 700 + 10 * b + rank)).cuda()
            t.populate_cache(k)
        t.use_cache = True
        ref_out = out.clone()
        t.use_cache = False
        step(0)
        torch.cuda.synchronize()
        ref_out.copy_(out)
        t.use_cache = True
        t.cache_misses(reset=True)
        step(0)
        misses = t.cache_misses(reset=True)
        same = bool(torch.equal(out, ref_out))
        sec_c = timed()
        hit = 1.0 - misses / n
        res["with_cache"] = {"cache_frac_of_shard": cache_frac, "hit_rate": hit, "same_output": same,
                             "keys_per_s": n * world / sec_c, "ms_per_step": sec_c * 1e3,
                             "nvlink_gbs_per_rank": misses * row_bytes * (world - 1) / max(world, 1) / sec_c / 1e9}
    t.close()
    return res
