"""Benchmark drivers beside bench.py: the clock sampler and timing helpers the benchmark shares, the
records that bench.py adds to its JSON line for the other configurations (sharded table at every
world size; int8 dequantise + pool, gradient de-duplication + update and the cached host-table
gather on single-GPU runs), and the stand-alone runs of those configurations

    python bench.py --workload c3|c4a|c4b|c5|published [--steps K] [--warmup W]

Each function builds seeded synthetic inputs of the configuration's shape on the current CUDA device
and times the path with CUDA events on the launching stream.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from nv_embedding_cache_b200 import capi, datagen as dg                                     # noqa: E402
from nv_embedding_cache_b200.layers import GpuTable, GPUEmbeddingLayer, LinearUVMEmbeddingLayer  # noqa: E402


class ClockSampler:
    """Samples SM clocks / throttle reasons while a timed region runs: a background thread polls
    and `sample_now()` takes one more reading while the queued work of the region is still
    executing.  NVML in-process when the binding is there (a query is a few microseconds and touches
    one device); otherwise one nvidia-smi process per sample."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid: str | None = None, period_s: float = 0.05):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.rows = []
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        self._handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            if uuid:
                try:
                    self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
                except Exception:
                    self._handle = None
            if self._handle is None:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    @classmethod
    def for_current_device(cls, period_s: float = 0.05):
        dev = torch.cuda.current_device()
        uuid = str(getattr(torch.cuda.get_device_properties(dev), "uuid", "") or "")
        return cls(dev, uuid, period_s)

    def _sample_nvml(self):
        n, h = self._nvml, self._handle
        sm = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
        try:
            power = n.nvmlDeviceGetPowerUsage(h) / 1000.0
        except Exception:
            power = 0.0
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            n.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = int(get(h))
        flag = lambda mask: "Active" if bits & mask else "Not Active"   # NVML reason bits
        return [str(sm), str(mx), f"{power:.1f}", flag(0x8), flag(0x40), flag(0x20), flag(0x4)]

    def sample_now(self):
        try:
            if self._nvml is not None:
                row = self._sample_nvml()
                with self._lock:
                    self.rows.append(row)
                return
            out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}",
                                  "--format=csv,noheader,nounits", "-i", str(self.gpu_index)],
                                 capture_output=True, text=True, timeout=10).stdout.strip()
            if out:
                with self._lock:
                    self.rows.append([x.strip() for x in out.splitlines()[0].split(",")])
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self.sample_now()
            self._stop.wait(self.period_s if self._nvml is not None else 0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=15)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def hbm_peak(root=ROOT):
    p = Path(root) / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _hbm_peak(root):
    return hbm_peak(root)


def world_info():
    import torch.distributed as dist
    if dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def barrier():
    import torch.distributed as dist
    torch.cuda.synchronize()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize()


def reduce_max(x: float) -> float:
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def reduce_sum(x: float) -> float:
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def timed_repeats(stream, fn, steps: int, warmup: int, repeats: int = 5):
    """`repeats` timed regions of exactly `steps` calls of fn(i) each, after `warmup` untimed calls:
    every region is bracketed by a barrier and a device synchronisation on both sides and timed
    with CUDA events on `stream`; a region's time is the maximum over the ranks.  Returns
    (median milliseconds per region, all regions' milliseconds)."""
    for i in range(warmup):
        fn(i)
    it = warmup
    regions = []
    for _ in range(repeats):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn(it)
            it += 1
        e1.record(stream)
        barrier()
        regions.append(reduce_max(e0.elapsed_time(e1)))
    return float(np.median(regions)), regions


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


def cpu_timed(fn, seconds: float, min_calls: int = 3, max_calls: int = 200):
    """Wall-clock times of fn() on the host for about `seconds`: (median s, mean s, calls)."""
    fn()
    times = []
    t_end = time.perf_counter() + seconds
    while len(times) < min_calls or (time.perf_counter() < t_end and len(times) < max_calls):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return float(np.median(times)), float(np.mean(times)), len(times)


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
        from nv_embedding_cache_b200.memblock import ManagedMemBlock
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


# ---- the sharded table (at every world size) ------------------------------------------------------
def touched_rows_mirror(keys_np: np.ndarray, width: int, seed: int):
    """Host mirror of the rows a batch touches, regenerated from the table's counter hash (no read
    of device memory), and the keys re-indexed into it."""
    uniq, inv = np.unique(keys_np, return_inverse=True)
    rows = dg.hashed_rows_f16(uniq, width, seed)
    return rows.view(np.uint8).reshape(uniq.size, -1), inv.astype(np.int64)


def sharded_record(steps=20, warmup=5, repeats=5, rows_per_rank=250_000_000, dim=64, bags=131_072, hot=8,
                   sample_batches=80, hot_capacity=20_000_000, modes=("peer", "peer_hot", "alltoall_hot"),
                   table_seed=60):
    """The NVLink-sharded configuration: one table of rows_per_rank x W rows x 64 fp16 (32 GB per
    GPU), row r on rank r mod W; per rank 131 072 bags x 8 int64 keys, Zipf(1.05) over a permuted row
    order, sum pooled in fp32 to fp16.  Every form is timed as the median of `repeats` regions of
    `steps` lookups (max over ranks) and its first batch is compared bit for bit, on rank 0, with the
    oracle working on a host mirror of the touched rows.

      peer          one fused kernel, every row read from its owner (plain loads over NVLink)
      peer_hot      the same behind the replicated hot-row table, chosen from `sample_batches`
                    earlier batches of the key stream
      alltoall_hot  hash dedup -> keys to owners -> rows back (ncclSend/ncclRecv issued by the
                    library), hot keys served locally
      alltoall      the exchange form without hot rows (stand-alone runs)
    """
    from nv_embedding_cache_b200.sharded import ShardedEmbeddingTable, allocate_symmetric_shard
    from oracle.pyoracle import Oracle
    world, rank = world_info()
    stream = torch.cuda.current_stream()
    total = rows_per_rank * world
    n = bags * hot
    row_bytes = dim * 2
    t_setup = time.perf_counter()
    if world > 1:
        shard = allocate_symmetric_shard(rows_per_rank, dim, torch.float16)
    else:
        shard = torch.empty((rows_per_rank, dim), dtype=torch.float16, device="cuda")
    dg.fill_hashed_rows_f16(shard, first_row=rank, row_step=world, seed=table_seed)
    nb = 4
    keys_np = [dg.zipf_keys(n, total, 1.05, 600 + 10 * b + rank) for b in range(nb)]
    batches = [torch.from_numpy(k).cuda() for k in keys_np]
    sample_np = np.concatenate([dg.zipf_keys(n, total, 1.05, 900 + 50 * rank + b) for b in range(sample_batches)])
    sample = torch.from_numpy(sample_np).cuda()
    out = torch.empty((bags, dim), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    want = None
    if rank == 0:
        mirror, local = touched_rows_mirror(keys_np[0], dim, table_seed)
        want = Oracle().lookup_pooled(mirror, "f16", dim, local, "sum", hotness=hot, out_dtype="f16")
    # what the hot table holds: every distinct key of the sample when they fit (they do at the default sizes)
    sample_keys = np.unique(sample_np)
    hot_known = sample_keys.size <= hot_capacity
    res = {"workload": "C5 NVLink-sharded table: 250M x W rows x 64 fp16 (32 GB per GPU), row r on rank r mod W; "
                       "per rank 131072 bags x 8 int64 keys, Zipf(1.05), sum pooled in fp32 -> fp16",
           "n_gpus": world, "rows_per_rank": rows_per_rank, "keys_per_step_per_rank": n,
           "unique_keys_per_rank": int(np.unique(keys_np[0]).size), "steps": steps, "repeats": repeats,
           "setup_s": round(setup_s, 1), "hot_sample_batches": sample_batches, "hot_capacity_rows": hot_capacity,
           "scaling": "weak", "modes": {}}
    tables = {}
    with ClockSampler.for_current_device() as clk:
        for mode in modes:
            form = "peer" if mode.startswith("peer") else "alltoall"
            with_hot = mode.endswith("_hot")
            key = (form, with_hot)
            t = ShardedEmbeddingTable(shard, max_keys=n, mode=form, hot_rows=hot_capacity if with_hot else 0)
            tables[key] = t
            hot_rows = t.set_hot_keys(sample) if with_hot else 0

            def step(i, t=t):
                t.lookup_pooled(batches[i % nb], "sum", fixed_hotness=hot, out=out)
            out.zero_()
            step(0)
            torch.cuda.synchronize()
            parity = bool(np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))) if rank == 0 else None
            ms, regions = timed_repeats(stream, step, steps, warmup, repeats)
            clk.sample_now()
            sec = ms * 1e-3 / steps
            entry = {"keys_per_s": n * world / sec, "ms_per_step": sec * 1e3, "parity": parity,
                     "region_ms": [round(r, 4) for r in regions], "hot_rows": int(hot_rows)}
            if form == "peer":
                k0 = keys_np[0]
                served_locally = np.isin(k0, sample_keys) if (with_hot and hot_known) else np.zeros(k0.size, bool)
                remote = int(np.count_nonzero(~served_locally & (k0 % world != rank)))
                entry["hot_hit_rate"] = float(served_locally.mean()) if with_hot and hot_known else (None if with_hot else 0.0)
                entry["nvlink_bytes_in_per_step"] = remote * row_bytes
                entry["nvlink_gbs_per_rank"] = remote * row_bytes / sec / 1e9
            else:
                ex = dict(t.last_exchange)
                entry["unique_sent"] = ex.get("unique")
                entry["served"] = ex.get("served")
                entry["nvlink_bytes_out_per_step"] = ex.get("nvlink_bytes_out")
                entry["nvlink_gbs_per_rank"] = (ex.get("nvlink_bytes_out") or 0) / sec / 1e9
            # device bytes one lookup must move on this rank: keys, every row once, the pooled rows
            alg = n * (8 + row_bytes) + bags * row_bytes
            entry["algorithmic_gbs_per_rank"] = alg / sec / 1e9
            res["modes"][mode] = entry
    res["clocks"] = clk.summary()
    for t in tables.values():
        t.close()
    peak, kind = hbm_peak()
    res["hbm_peak_gbs"], res["peak_kind"] = peak, kind
    # parity over all ranks' view: rank 0 checked its batch; the flag is reduced so every rank agrees
    ok = all(m["parity"] for m in res["modes"].values()) if rank == 0 else True
    res["parity"] = bool(reduce_sum(0.0 if ok else 1.0) == 0.0)
    del shard
    torch.cuda.empty_cache()
    return res


def run_c5(root, steps=30, warmup=5, rows_per_rank=250_000_000, **kw):
    modes = tuple(os.environ.get("NVE_B200_SHARD_MODES", "peer,peer_hot,alltoall_hot,alltoall").split(","))
    extra = {}
    if os.environ.get("NVE_B200_SHARD_SAMPLE"):          # batches of the key sample the hot rows are chosen from
        extra["sample_batches"] = int(os.environ["NVE_B200_SHARD_SAMPLE"])
    if os.environ.get("NVE_B200_SHARD_HOT"):             # capacity of the hot-row table, in rows
        extra["hot_capacity"] = int(os.environ["NVE_B200_SHARD_HOT"])
    return sharded_record(steps=steps, warmup=warmup, rows_per_rank=rows_per_rank, modes=modes, **extra)


# ---- records of the single-GPU configurations for bench.py's JSON line --------------------------------
def _pinned(t: torch.Tensor) -> torch.Tensor:
    return t.cpu().pin_memory()


def _roofline(alg_bytes, sec, kernel, traffic_file=None):
    peak, kind = hbm_peak()
    r = {"bound": "hbm", "kernel": kernel, "achieved": alg_bytes / sec / 1e9, "peak": peak, "peak_kind": kind,
         "unit": "GB/s", "frac": alg_bytes / sec / 1e9 / peak, "traffic": None,
         "algorithmic_bytes_per_step": int(alg_bytes)}
    if traffic_file is not None:
        f = ROOT / "profiles" / traffic_file
        if f.exists():
            r["traffic"] = json.loads(f.read_text()).get("dram_bytes_per_launch")
    return r


def record_c4a(steps=20, warmup=5, repeats=5, rows=50_000_000, width=256, bags=32_768, hot=20, cpu_seconds=6.0):
    """find_and_dequant + sum pooling: 50M x 256 int8 with a per-row fp32 scale stored right after
    the values (260-byte rows), 32768 bags x 20 int64 keys Zipf(1.05), fp32 sums -> fp16."""
    stream = torch.cuda.current_stream()
    stride = width + 4
    nb = 4
    keys_np = [dg.zipf_keys(bags * hot, rows, 1.05, 400 + b) for b in range(nb)]
    batches = [torch.from_numpy(k).cuda() for k in keys_np]
    n = bags * hot
    out = torch.empty((bags, width), dtype=torch.float16, device="cuda")
    t = _quant_table(rows, width, stride, 40)
    a = capi.PoolArgs()
    a.table, a.num_rows, a.row_stride = t.data_ptr(), rows, stride
    a.value_dtype, a.row_width, a.default_row_index = capi.DTYPE_QINT8_F32, width, -1
    a.cache, a.key_type, a.num_keys = None, capi.KEY_INT64, n
    a.pooling_type, a.sparse_type, a.num_bags, a.fixed_hotness = capi.POOL_SUM, capi.SPARSE_FIXED, bags, hot
    a.output, a.output_stride, a.output_dtype = out.data_ptr(), width * 2, capi.DTYPE_FLOAT16

    def launch(i):
        a.keys = batches[i % nb].data_ptr()
        capi.check(capi.lib.nve_b200_lookup_pool(C.byref(a), stream.cuda_stream))
    # end to end: pinned host keys in, pooled rows out to pinned host memory
    pin_keys = [torch.from_numpy(k).pin_memory() for k in keys_np]
    dev_keys = torch.empty(n, dtype=torch.int64, device="cuda")
    pin_out = torch.empty((bags, width), dtype=torch.float16).pin_memory()

    def launch_e2e(i):
        dev_keys.copy_(pin_keys[i % nb], non_blocking=True)
        a.keys = dev_keys.data_ptr()
        capi.check(capi.lib.nve_b200_lookup_pool(C.byref(a), stream.cuda_stream))
        pin_out.copy_(out, non_blocking=True)
    with ClockSampler.for_current_device() as clk:
        ms, regions = timed_repeats(stream, launch, steps, warmup, repeats)
        clk.sample_now()
        ms_e2e, _ = timed_repeats(stream, launch_e2e, steps, warmup, 3)
    sec = ms * 1e-3 / steps
    alg = n * (8 + stride) + bags * width * 2
    rec = {"workload": "C4a: 50M x 256 int8 + fp32 scale (260-byte rows), 32768 bags x 20 keys Zipf(1.05), dequant + sum -> fp16",
           "keys_per_s": n / sec, "us_per_step": sec * 1e6, "region_ms": [round(r, 4) for r in regions],
           "roofline": _roofline(alg, sec, "pool_dense_kernel<I8,GROUP=16,U=4,WORDS>", "pool_dense_i8_c4a.traffic.json"),
           "clocks": clk.summary(),
           "e2e": {"value": n / (ms_e2e * 1e-3 / steps), "unit": "keys/s", "h2d_bytes_per_step": n * 8,
                   "d2h_bytes_per_step": bags * width * 2}}
    # CPU baseline: the reference host layer on a table of identical row size, sub-sampled in rows
    try:
        from oracle.pyoracle import Reference
        sub = 2_000_000
        host = dg.quantized_rows(sub, width, 41, "qint8_f32", stride)
        layer = Reference(for_timing=True).layer(host, "qint8_f32")
        hk = (keys_np[0] % sub).astype(np.int64)
        hout = np.zeros((bags, width), np.float16)
        med, mean, calls = cpu_timed(lambda: layer.lookup_pooled(hk, "sum", width, hotness=hot, out_dtype="f16", out=hout),
                                     cpu_seconds)
        rec["cpu_baseline"] = {"value": n / med, "unit": "keys/s", "cores": int(layer.num_workers), "kind": "reference",
                               "sample": f"{calls} pooled lookups of the batch on a {sub}-row host table of the same "
                                         f"260-byte rows (keys mod {sub}); median {med * 1e3:.1f} ms, mean {mean * 1e3:.1f} ms"}
        layer.close()
    except Exception as e:      # noqa: BLE001 - the checker library is absent: report, do not fake
        rec["cpu_baseline"] = {"value": None, "unit": "keys/s", "cores": 0, "kind": "reference", "sample": f"unavailable: {e}"}
    del t
    torch.cuda.empty_cache()
    return rec


def record_c4b(steps=10, warmup=3, repeats=5, rows=10_000_000, dim=128, n=1_048_576, lr=0.01, cpu_seconds=6.0):
    """dedup_grads + update_accumulate: 1 048 576 (int64 key Zipf(1.05), fp32 grad N(0, 1e-2)) pairs into
    a 10M x 128 fp32 table, SGD lr 0.01."""
    stream = torch.cuda.current_stream()
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
    src_keys = {"ptr": keys.data_ptr()}
    src_grads = {"ptr": grads.data_ptr()}

    def dedup(i):
        capi.check(capi.lib.nve_b200_deduper_dedup(d, src_keys["ptr"], n, uniq.data_ptr(), counts.data_ptr(),
                                                   loc.data_ptr(), None, inverse.data_ptr(), offsets.data_ptr(), s, 24))

    def apply(i):
        capi.check(capi.lib.nve_b200_dedup_grads(d, src_grads["ptr"], dim * 4, dim * 4, n, uniq.data_ptr(),
                                                 inverse.data_ptr(), offsets.data_ptr(), loc.data_ptr(),
                                                 table.data_ptr(), dim * 4, 1, rows, -lr, s))

    def both(i):
        dedup(i)
        apply(i)
    pin_keys = torch.from_numpy(keys_np).pin_memory()
    pin_grads = _pinned(grads)
    dev_keys = torch.empty_like(keys)
    dev_grads = torch.empty_like(grads)
    pin_done = torch.zeros(8, dtype=torch.int64).pin_memory()

    def both_e2e(i):
        dev_keys.copy_(pin_keys, non_blocking=True)
        dev_grads.copy_(pin_grads, non_blocking=True)
        src_keys["ptr"], src_grads["ptr"] = dev_keys.data_ptr(), dev_grads.data_ptr()
        both(i)
        pin_done.copy_(uniq[:8], non_blocking=True)      # the step's result read back: a handful of unique keys
        src_keys["ptr"], src_grads["ptr"] = keys.data_ptr(), grads.data_ptr()
    capi.check(capi.lib.nve_b200_deduper_dedup(d, keys.data_ptr(), n, uniq.data_ptr(), counts.data_ptr(), loc.data_ptr(),
                                               runs, inverse.data_ptr(), offsets.data_ptr(), s, 24))
    u = int(runs[0])
    with ClockSampler.for_current_device() as clk:
        ms_dedup, _ = timed_repeats(stream, dedup, steps, warmup, repeats)
        ms_apply, _ = timed_repeats(stream, apply, steps, warmup, repeats)
        ms, regions = timed_repeats(stream, both, steps, warmup, repeats)
        clk.sample_now()
        ms_e2e, _ = timed_repeats(stream, both_e2e, max(2, steps // 2), 2, 3)
    sec = ms * 1e-3 / steps
    alg = n * (8 + dim * 4) + u * 2 * dim * 4
    rec = {"workload": "C4b: dedup_grads + update_accumulate, 1048576 (key, grad) pairs Zipf(1.05), 10M x 128 fp32, SGD lr 0.01",
           "unique": u, "keys_per_s": n / sec, "us_per_step": sec * 1e6, "us_dedup": ms_dedup * 1e3 / steps,
           "us_reduce_apply": ms_apply * 1e3 / steps, "region_ms": [round(r, 4) for r in regions],
           "roofline": _roofline(alg, sec, "dedup (sort + emit) + grad_stream_kernel/grad_heavy_kernel (fused apply)"),
           "clocks": clk.summary(),
           "e2e": {"value": n / (ms_e2e * 1e-3 / max(2, steps // 2)), "unit": "keys/s",
                   "h2d_bytes_per_step": n * (8 + dim * 4), "d2h_bytes_per_step": 64}}
    capi.check(capi.lib.nve_b200_deduper_destroy(d))
    try:
        from oracle.pyoracle import Reference
        sub = 1_000_000
        host = np.zeros((sub, dim), np.float32)
        layer = Reference(for_timing=True).layer(host.view(np.uint8).reshape(sub, dim * 4), "f32")
        hk_all = (keys_np % sub).astype(np.int64)
        hg = grads[:n].cpu().numpy()

        def cpu_step():
            # the reference's CPU path for this work: coalesce the pairs (numpy stands in for its
            # caller-side dedup), then cpu_kernel_update_accumulate through the host layer
            order = np.argsort(hk_all, kind="stable")
            uk, first = np.unique(hk_all[order], return_index=True)
            sums = np.add.reduceat(hg[order], first, axis=0) * np.float32(-lr)
            layer.accumulate(uk, sums)
        med, mean, calls = cpu_timed(cpu_step, cpu_seconds, min_calls=2, max_calls=20)
        rec["cpu_baseline"] = {"value": n / med, "unit": "keys/s", "cores": int(layer.num_workers), "kind": "reference",
                               "sample": f"{calls} steps: numpy stable sort + segmented sum of the {n} pairs (single thread), then the "
                                         f"reference host layer's accumulate of the unique rows into a {sub}-row fp32 table; "
                                         f"median {med * 1e3:.0f} ms, mean {mean * 1e3:.0f} ms"}
        layer.close()
    except Exception as e:      # noqa: BLE001
        rec["cpu_baseline"] = {"value": None, "unit": "keys/s", "cores": 0, "kind": "reference", "sample": f"unavailable: {e}"}
    del table, grads, dev_grads
    torch.cuda.empty_cache()
    return rec


def record_c3(steps=20, warmup=5, repeats=5, rows=100_000_000, dim=128, batch=262_144, cache_frac=0.10,
              cpu_seconds=5.0):
    """LinearUVM cached un-pooled lookup: 100M x 128 fp16 (25.6 GB) in a managed block kept in host
    memory, 10 % of the rows cached on the GPU after 20 insert batches; 262 144 int64 keys per lookup,
    Zipf(1.2) and a uniform (miss-heavy) run."""
    from nv_embedding_cache_b200.memblock import ManagedMemBlock
    row_bytes = dim * 2
    stream = torch.cuda.current_stream()
    block = ManagedMemBlock(rows * row_bytes, (torch.cuda.current_device(),))
    table = block.as_tensor((rows, dim), torch.float16)
    _fill_rows_fp16(table, 30)
    gt = GpuTable(int(rows * cache_frac) * row_bytes, row_bytes, "float16", uvm_table=table, uvm_num_rows=rows)
    layer = LinearUVMEmbeddingLayer(gt)
    ctx = layer.create_execution_context(stream.cuda_stream, stream.cuda_stream)
    for b in range(20):
        k = torch.from_numpy(dg.zipf_keys(batch, rows, 1.2, 300 + b)).cuda()
        capi.check(capi.lib.nve_b200_gpu_table_insert_from_backing(gt.handle, ctx.handle, batch, k.data_ptr()))
    ctx.wait()
    out = torch.empty((batch, dim), dtype=torch.float16, device="cuda")
    link = h2d_probe_gbs(1 << 30, 5)
    nb = 16
    rec = {"workload": "C3 LinearUVM: 100M x 128 fp16 in host memory (managed block), 10% GPU cache warmed by 20 inserts, "
                       "262144 int64 keys per un-pooled lookup", "host_link_probe_gbs": link, "runs": {}}
    with ClockSampler.for_current_device() as clk:
        for name, gen_keys in (("zipf1.2", lambda b: dg.zipf_keys(batch, rows, 1.2, 320 + 2 * b)),
                               ("uniform", lambda b: dg.uniform_keys(batch, rows, 321 + 2 * b))):
            keys_np = [gen_keys(b) for b in range(nb)]
            batches = [torch.from_numpy(k).cuda() for k in keys_np]
            hr = layer.lookup(ctx, batch, batches[0], out, row_bytes, want_hitrate=True)
            ctx.wait()
            exact = bool(torch.equal(out.cpu(), table[torch.from_numpy(keys_np[0])]))
            ms, regions = timed_repeats(stream, lambda i: layer.lookup(ctx, batch, batches[i % nb], out, row_bytes),
                                        steps, warmup, repeats)
            clk.sample_now()
            sec = ms * 1e-3 / steps
            misses = round((1.0 - hr) * batch)
            pin_keys = [torch.from_numpy(k).pin_memory() for k in keys_np[:4]]
            pin_out = torch.empty((batch, dim), dtype=torch.float16).pin_memory()
            ms_e2e, _ = timed_repeats(stream, lambda i: layer.lookup(ctx, batch, pin_keys[i % 4], pin_out, row_bytes),
                                      max(4, steps // 2), 2, 3)
            alg = batch * (8 + 2 * row_bytes)
            rec["runs"][name] = {
                "keys_per_s": batch / sec, "us_per_step": sec * 1e6, "hit_rate": hr, "byte_exact": exact,
                "region_ms": [round(r, 4) for r in regions],
                "roofline": _roofline(alg, sec, "lookup_rows_kernel (cache probe + row copy)"),
                "host_link_gbs": misses * row_bytes / sec / 1e9,
                "host_link_frac_of_probe": misses * row_bytes / sec / 1e9 / link,
                "e2e": {"value": batch / (ms_e2e * 1e-3 / max(4, steps // 2)), "unit": "keys/s",
                        "h2d_bytes_per_step": batch * 8, "d2h_bytes_per_step": batch * row_bytes}}
        # pooled lookups through the same cache (the cached layer's find_and_pool): 32768 bags x 8 keys, sum
        bags, hot = 32_768, 8
        pk_np = [dg.zipf_keys(bags * hot, rows, 1.2, 360 + b) for b in range(4)]
        pk = [torch.from_numpy(k).cuda() for k in pk_np]
        out_p = torch.empty((bags, dim), dtype=torch.float16, device="cuda")
        hr_p = layer.lookup_pooled(ctx, bags * hot, pk[0], out_p, row_bytes, "sum", "float16", fixed_hotness=hot,
                                   want_hitrate=True)
        ctx.wait()
        uniq, inv = np.unique(pk_np[0], return_inverse=True)
        mirror = table[torch.from_numpy(uniq)].numpy()
        from oracle.pyoracle import Oracle
        want = Oracle().lookup_pooled(mirror.view(np.uint8).reshape(uniq.size, -1), "f16", dim, inv.astype(np.int64),
                                      "sum", hotness=hot, out_dtype="f16")
        same = bool(np.array_equal(out_p.cpu().numpy().view(np.uint16), want.view(np.uint16)))
        ms_p, _ = timed_repeats(stream, lambda i: layer.lookup_pooled(ctx, bags * hot, pk[i % 4], out_p, row_bytes, "sum",
                                                                      "float16", fixed_hotness=hot),
                                steps, warmup, repeats)
        sec_p = ms_p * 1e-3 / steps
        alg_p = bags * hot * (8 + row_bytes) + bags * row_bytes
        rec["pooled"] = {"workload": "32768 bags x 8 Zipf(1.2) keys, sum pooled through the cache (find_and_pool)",
                         "keys_per_s": bags * hot / sec_p, "us_per_step": sec_p * 1e6, "hit_rate": hr_p, "bit_exact": same,
                         "roofline": _roofline(alg_p, sec_p, "shard_pool_kernel (cache line or table row per key)")}
        try:
            from oracle.pyoracle import ReferenceGpu
            rg = ReferenceGpu()
            rc = rg.cache(int(rows * cache_frac) * row_bytes, row_bytes, max_modify=batch)
            for b in range(20):
                k = torch.from_numpy(dg.zipf_keys(batch, rows, 1.2, 300 + b)).cuda()
                rc.insert_from_table(k.data_ptr(), batch, table.data_ptr(), row_bytes)
            torch.cuda.synchronize()
            ms_r = rc.find_and_combine(bags, table.data_ptr(), [k.data_ptr() for k in pk], hot, dim, out_p.data_ptr(),
                                       warmup=warmup, iters=steps)
            rec["pooled"]["reference_gpu_kernel"] = {
                "kernel": "find_and_combine with the reference cache in front (same inserts, same batches)",
                "us_per_step": ms_r * 1e3, "keys_per_s": bags * hot / (ms_r * 1e-3)}
            rc.close()
        except Exception as e:      # noqa: BLE001 - the reference GPU library is absent: say so
            rec["pooled"]["reference_gpu_kernel"] = {"unavailable": str(e)[:200]}
    rec["clocks"] = clk.summary()
    try:
        from oracle.pyoracle import Reference
        sub = 4_000_000
        host = table[:sub].numpy().view(np.uint8).reshape(sub, row_bytes)
        ref_layer = Reference(for_timing=True).layer(np.ascontiguousarray(host), "f16")
        hk = (dg.zipf_keys(batch, rows, 1.2, 320) % sub).astype(np.int64)
        hout = np.zeros((batch, dim), np.float16)
        med, mean, calls = cpu_timed(lambda: ref_layer.lookup(hk, hout), cpu_seconds)
        rec["cpu_baseline"] = {"value": batch / med, "unit": "keys/s", "cores": int(ref_layer.num_workers), "kind": "reference",
                               "sample": f"{calls} un-pooled lookups of the Zipf batch through the reference host layer on the "
                                         f"first {sub} rows of the same table (keys mod {sub}; the CPU layer has no cache); "
                                         f"median {med * 1e3:.2f} ms, mean {mean * 1e3:.2f} ms"}
        ref_layer.close()
    except Exception as e:      # noqa: BLE001
        rec["cpu_baseline"] = {"value": None, "unit": "keys/s", "cores": 0, "kind": "reference", "sample": f"unavailable: {e}"}
    ctx.destroy(); layer.destroy(); gt.destroy()
    del table
    block.close()
    torch.cuda.empty_cache()
    return rec


def copy_probe(nbytes=256 << 20, reps=5):
    """Pinned-memory copies by every rank at once, host -> device and device -> host on two streams
    (plain cudaMemcpyAsync through torch): what the box's host side gives all GPUs together, next to
    which the end-to-end figures of multi-rank runs are read.  Returns GB/s of this rank and summed
    over the ranks."""
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    d_out = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    s0, s1 = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    best = None
    for _ in range(reps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        s0.wait_stream(main)
        s1.wait_stream(main)
        with torch.cuda.stream(s0):
            d_in.copy_(h_in, non_blocking=True)
        with torch.cuda.stream(s1):
            h_out.copy_(d_out, non_blocking=True)
        main.wait_stream(s0)
        main.wait_stream(s1)
        e1.record(main)
        barrier()
        ms = reduce_max(e0.elapsed_time(e1))
        best = ms if best is None else min(best, ms)
    world, _ = world_info()
    per_rank = 2 * nbytes / (best * 1e-3) / 1e9
    return {"bytes_each_way": nbytes, "gbs_per_rank_both_ways": per_rank, "gbs_all_ranks_both_ways": per_rank * world,
            "note": "all ranks copy at once; time is the slowest rank's"}
