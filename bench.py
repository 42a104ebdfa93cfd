#!/usr/bin/env python
"""Benchmark of the embedding lookup hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config "GPULayer, fully HBM-resident"): 8 independent tables of 4,000,000 rows x
128 fp16 (N(0, 0.02)); per table 65,536 bags of 1..32 int64 keys, Zipf(1.1) over a permuted row
order, CSR offsets, mean pooling accumulated in fp32, output [65536,128] fp16.  One *step* is one
pooled lookup of every table (8 launches of the fused gather+pool kernel).  Tables and key batches
are seeded synthetic data.  With N > 1 every rank serves its own 8 tables (independent tables: no
data-path collective, weak scaling).

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NUM_TABLES = 8
NUM_ROWS = 4_000_000
WIDTH = 128
ROW_BYTES = WIDTH * 2
NUM_BAGS = 65_536
ALPHA = 1.1
NUM_BATCHES = 4          # distinct key batches per table, cycled over the steps
METRIC = "embedding keys/sec (find-and-combine)"
WORKLOAD = "C2 GPULayer HBM-resident: 8 tables x 4M x 128 fp16, 65536 CSR bags len U[1,32], Zipf(1.1), mean pool fp32 acc"


def make_batch(table_idx: int, batch_idx: int, rank: int, perm: np.ndarray):
    from nv_embedding_cache_b200 import datagen as dg
    seed = 1000 + 200 + 10 * table_idx + batch_idx + 1000 * rank
    _, offsets = dg.csr_bags(NUM_BAGS, 1, 32, seed)
    keys = dg.zipf_keys(int(offsets[-1]), NUM_ROWS, ALPHA, seed + 5000, perm)
    return keys, offsets


def algorithmic_bytes(num_keys: int) -> int:
    """Bytes one pooled lookup must move: keys + rows read, offsets read, pooled rows written."""
    return num_keys * (8 + ROW_BYTES) + (NUM_BAGS + 1) * 8 + NUM_BAGS * ROW_BYTES


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs: a background
    thread polls continuously and `sample_now()` takes one more reading while the queued work of
    the region is still executing."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid: str | None = None):
        self.gpu_index = gpu_index
        self.rows = []
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        # NVML in-process when the binding is there (a query is a few microseconds and touches one
        # device); otherwise one nvidia-smi process per sample.
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
            self._stop.wait(0.2)

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


def measured_hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def cpu_reference_run(table_host: np.ndarray, batches, seconds_budget: float, min_calls: int = 3):
    """Times the reference CPU implementation (HostEmbeddingLayer over a LinearHostTable, the
    unmodified reference sources built into oracle/_ref) on one table's pooled lookups."""
    from oracle.pyoracle import Reference
    ref = Reference()
    layer = ref.layer(table_host.view(np.uint8).reshape(NUM_ROWS, ROW_BYTES), "f16")
    workers = layer.num_workers
    out = np.zeros((NUM_BAGS, WIDTH), dtype=np.float16)
    keys, offsets = batches[0]
    layer.lookup_pooled(keys, "mean", WIDTH, offsets=offsets, out_dtype="f16", out=out)  # warm-up
    times, total_keys, i = [], 0, 0
    t_end = time.perf_counter() + seconds_budget
    while len(times) < min_calls or time.perf_counter() < t_end:
        keys, offsets = batches[i % len(batches)]
        t0 = time.perf_counter()
        layer.lookup_pooled(keys, "mean", WIDTH, offsets=offsets, out_dtype="f16", out=out)
        times.append(time.perf_counter() - t0)
        total_keys += keys.size
        i += 1
        if len(times) >= 200:
            break
    layer.close()
    return total_keys / sum(times), workers, len(times), float(np.median(times))


def load_reference_gpu():
    """The unmodified reference GPU code built into oracle/_ref (a baseline timed beside this
    library's kernels, never on their path); None when the library was not built."""
    try:
        from oracle.pyoracle import ReferenceGpu
        return ReferenceGpu()
    except (FileNotFoundError, OSError):
        return None


def run_reference_arm(args):
    """--impl reference: the reference's own CPU path on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from nv_embedding_cache_b200 import datagen as dg
    perm = dg.permutation(NUM_ROWS)
    table = dg.normal_table(NUM_ROWS, WIDTH, 0.02, 20, np.float16)
    batches = [make_batch(0, b, 0, perm) for b in range(NUM_BATCHES)]
    from oracle.pyoracle import Reference
    ref = Reference()
    layer = ref.layer(table.view(np.uint8).reshape(NUM_ROWS, ROW_BYTES), "f16")
    workers = layer.num_workers
    out = np.zeros((NUM_BAGS, WIDTH), dtype=np.float16)

    def step(i):
        keys, offsets = batches[i % NUM_BATCHES]
        layer.lookup_pooled(keys, "mean", WIDTH, offsets=offsets, out_dtype="f16", out=out)
        return keys.size

    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    nkeys = 0
    for i in range(args.steps):
        nkeys += step(i)
    dt = time.perf_counter() - t0
    layer.close()
    value = nkeys / dt
    sample = (f"each step = one table's pooled lookup ({batches[0][0].size} keys, 65536 bags) of the "
              f"8-table workload, {args.steps} steps")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "keys/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": value, "unit": "keys/s", "cores": int(workers),
                         "kind": "reference", "sample": sample, "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": "keys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nv_embedding_cache_b200 import capi, datagen as dg
    from nv_embedding_cache_b200.layers import GPUEmbeddingLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the lookup path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- tables (seeded, generated on the device) and key batches (seeded numpy)
    gen = torch.Generator(device=dev)
    tables = []
    for t in range(NUM_TABLES):
        gen.manual_seed(20 + t + 100 * rank)
        tab = torch.empty((NUM_ROWS, WIDTH), dtype=torch.float16, device=dev)
        chunk = 1 << 20
        for r0 in range(0, NUM_ROWS, chunk):
            r1 = min(NUM_ROWS, r0 + chunk)
            tab[r0:r1] = (torch.randn((r1 - r0, WIDTH), generator=gen, device=dev) * 0.02).half()
        tables.append(tab)
    perm = dg.permutation(NUM_ROWS)
    host_batches = [[make_batch(t, b, rank, perm) for b in range(NUM_BATCHES)]
                    for t in range(NUM_TABLES)]

    stream = torch.cuda.Stream(device=dev)
    # device-resident leg: every table on one stream (launches back to back);
    # end-to-end leg: one stream per table, so that the host->device copies of one table overlap
    # the device->host copies of another (the link is full duplex).
    table_streams = [torch.cuda.Stream(device=dev) for _ in range(NUM_TABLES)]
    layers, ctxs, ctxs_e2e = [], [], []
    for t in range(NUM_TABLES):
        layer = GPUEmbeddingLayer(tables[t], NUM_ROWS, ROW_BYTES, "float16", device_id=local_rank,
                                  layer_name=f"table{t}")
        layers.append(layer)
        ctxs.append(layer.create_execution_context(stream.cuda_stream, stream.cuda_stream))
        ctxs_e2e.append(layer.create_execution_context(table_streams[t].cuda_stream,
                                                       table_streams[t].cuda_stream))

    dev_batches = [[(torch.from_numpy(k).to(dev), torch.from_numpy(o).to(dev)) for k, o in hb]
                   for hb in host_batches]
    pin_batches = [[(torch.from_numpy(k).pin_memory(), torch.from_numpy(o).pin_memory())
                    for k, o in hb] for hb in host_batches]
    dev_out = [torch.empty((NUM_BAGS, WIDTH), dtype=torch.float16, device=dev)
               for _ in range(NUM_TABLES)]
    pin_out = [torch.empty((NUM_BAGS, WIDTH), dtype=torch.float16).pin_memory()
               for _ in range(NUM_TABLES)]

    def step_device(i):
        n = 0
        for t in range(NUM_TABLES):
            k, o = dev_batches[t][i % NUM_BATCHES]
            layers[t].lookup_pooled(ctxs[t], k.numel(), k, dev_out[t], ROW_BYTES, "mean", "float16",
                                    csr_offsets=o, num_csr_offsets=o.numel())
            n += k.numel()
        return n

    def step_host(i):
        n = hb = 0
        for t in range(NUM_TABLES):
            k, o = pin_batches[t][i % NUM_BATCHES]
            layers[t].lookup_pooled(ctxs_e2e[t], k.numel(), k, pin_out[t], ROW_BYTES, "mean",
                                    "float16", csr_offsets=o, num_csr_offsets=o.numel())
            n += k.numel()
            hb += k.numel() * 8 + o.numel() * 8
        return n, hb

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, fan_out):
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank, str(getattr(torch.cuda.get_device_properties(dev), "uuid", "") or "")) as clk:
            e0.record(stream)
            if fan_out:
                for ts in table_streams:
                    ts.wait_event(e0)
            keys = 0
            extra = 0
            for i in range(steps):
                r = fn(warmup + i)
                if isinstance(r, tuple):
                    keys += r[0]
                    extra += r[1]
                else:
                    keys += r
            if fan_out:
                for ts in table_streams:
                    ev = torch.cuda.Event()
                    ev.record(ts)
                    stream.wait_event(ev)
            e1.record(stream)
            clk.sample_now()   # the queue of this region is still draining
            barrier()
        ms = e0.elapsed_time(e1)
        return ms, keys, extra, clk.summary()

    # One step of the device-resident leg is eight short launches issued from Python, about as long
    # on the host as on the GPU.  Each of the four cycled steps is therefore captured once as a CUDA
    # graph and replayed (same kernels, same arguments); --no-graph, or a capture that fails, keeps
    # the direct launches.
    graphs = []
    # Single-rank runs only: with a NCCL process group alive in the process the capture was seen not
    # to complete on an 8-rank run, so multi-rank runs keep the direct launches.
    if not args.no_graph and world == 1:
        try:
            with torch.cuda.stream(stream):
                for b in range(NUM_BATCHES):
                    step_device(b)
                torch.cuda.synchronize()
                for b in range(NUM_BATCHES):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                        step_device(b)
                    graphs.append(g)
        except Exception as e:  # noqa: BLE001 - reported, then the direct path is used
            print(f"graph capture failed ({e!r}); launching directly", file=sys.stderr)
            graphs = []
            torch.cuda.synchronize()
    keys_of_step = [sum(k.numel() for k, _ in (dev_batches[t][b] for t in range(NUM_TABLES)))
                    for b in range(NUM_BATCHES)]

    def step_replay(i):
        graphs[i % NUM_BATCHES].replay()
        return keys_of_step[i % NUM_BATCHES]

    with torch.cuda.stream(stream):
        ms_dev, keys_dev, _, clocks = timed(step_replay if graphs else step_device, args.steps, args.warmup, False)
        ms_e2e, keys_e2e, h2d, _ = timed(step_host, args.steps, args.warmup, True)

    # ---- per-launch times outside the timed region (this rank): back-to-back launches, and launches
    # that each follow a 256 MB write, which leaves nothing of the tables or keys in L2
    def launch_times(flush):
        scrub = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None
        pairs = []
        for i in range(3):
            for t in range(NUM_TABLES):
                if scrub is not None:
                    scrub.fill_(i)
                k, o = dev_batches[t][i % NUM_BATCHES]
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                layers[t].lookup_pooled(ctxs[t], k.numel(), k, dev_out[t], ROW_BYTES, "mean", "float16",
                                        csr_offsets=o, num_csr_offsets=o.numel())
                b.record(stream)
                pairs.append((a, b))
        torch.cuda.synchronize()
        us = sorted(a.elapsed_time(b) * 1e3 for a, b in pairs[NUM_TABLES:])    # first round: warm-up
        return {"median_us": us[len(us) // 2], "min_us": us[0], "launches": len(us)}

    with torch.cuda.stream(stream):
        per_launch = {"back_to_back": launch_times(False), "cold_l2": launch_times(True)}

    # ---- max over ranks, whole-job totals
    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    ms_dev_max, ms_e2e_max = reduce_max(ms_dev), reduce_max(ms_e2e)
    keys_dev_all, keys_e2e_all = reduce_sum(keys_dev), reduce_sum(keys_e2e)
    value = keys_dev_all / (ms_dev_max * 1e-3)
    e2e_value = keys_e2e_all / (ms_e2e_max * 1e-3)

    # ---- roofline of the dominant kernel (this rank): algorithmic bytes per launch / mean launch time
    launches = args.steps * NUM_TABLES
    mean_launch_s = ms_dev * 1e-3 / launches
    alg_bytes = algorithmic_bytes(keys_dev // launches)
    peak, peak_kind = measured_hbm_peak()
    achieved = alg_bytes / mean_launch_s / 1e9
    roofline = {"bound": "hbm", "kernel": "pool_dense_kernel<F16,GROUP=16,U=4>",
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": achieved / peak, "traffic": None,
                "algorithmic_bytes_per_launch": alg_bytes, "mean_launch_us": mean_launch_s * 1e6}
    traffic_file = ROOT / "profiles" / "lookup_pool_f16_c2.traffic.json"
    if traffic_file.exists():
        roofline["traffic"] = json.loads(traffic_file.read_text()).get("dram_bytes_per_launch")

    out = {
        "metric": METRIC, "value": value, "unit": "keys/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev_max / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tables_per_gpu": NUM_TABLES,
                   "keys_per_step_per_gpu": keys_dev // args.steps,
                   "l2": "inputs larger than L2 (8.2 GB of tables, 4 key batches cycled)",
                   "launch": "CUDA graph of one step (8 kernels), replayed" if graphs else "direct launches",
                   "parallelism": f"replicas x{world} (independent tables, no collective)"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "keys/s",
                "h2d_bytes_per_step": h2d // args.steps,
                "d2h_bytes_per_step": NUM_TABLES * NUM_BAGS * ROW_BYTES,
                "ms_per_step": ms_e2e_max / args.steps},
        "gpu_launches": 2 * launches + 2 * args.warmup * NUM_TABLES,
        "roofline": roofline,
        "algo_bw_gib_s": value * ROW_BYTES / 2**30,
        "per_launch": per_launch,
    }

    # ---- CPU baseline beside it (rank 0, N=1 only): reference HostEmbeddingLayer on table 0
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            table_host = tables[0].cpu().numpy()
            v, workers, calls, med = cpu_reference_run(table_host, host_batches[0], args.cpu_seconds)
            out["cpu_baseline"] = {
                "value": v, "unit": "keys/s", "cores": int(workers), "kind": "reference",
                "host_cpus": os.cpu_count(),
                "sample": f"{calls} pooled lookups of table 0 ({host_batches[0][0][0].size} keys, "
                          f"65536 bags each; 1/8 of a step), median {med * 1e3:.1f} ms per lookup"}
        except Exception as e:  # the checker library is absent: report, do not fake
            out["cpu_baseline"] = {"value": None, "unit": "keys/s", "cores": 0, "kind": "reference",
                                   "sample": f"unavailable: {e}"}

    # ---- the reference's own GPU kernel for this lookup on the same GPU (rank 0, N=1 only):
    # find_and_combine reading the table directly, timed on table 0's four batches
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ref_gpu = load_reference_gpu()
        if ref_gpu is None:
            out["reference_gpu_kernel"] = {"unavailable": "oracle/_ref/libnve_ref_gpu.so is not built"}
        else:
            torch.cuda.synchronize()
            ks = [k.data_ptr() for k, _ in dev_batches[0]]
            os_ = [o.data_ptr() for _, o in dev_batches[0]]
            ms = ref_gpu.find_and_combine("f16_csr_mean", NUM_BAGS, tables[0].data_ptr(), ks, os_, 0, WIDTH,
                                          dev_out[0].data_ptr(), warmup=10, iters=100)
            nk = float(np.mean([k.numel() for k, _ in dev_batches[0]]))
            out["reference_gpu_kernel"] = {
                "kernel": "find_and_combine (fp16, CSR, mean, no cache in front), unmodified reference code",
                "us_per_launch": ms * 1e3, "value": nk / (ms * 1e-3), "unit": "keys/s",
                "sample": "table 0, 4 batches cycled, 100 launches"}

    for c in ctxs + ctxs_e2e:
        c.wait()
        c.destroy()
    for layer in layers:
        layer.destroy()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_other_workload(args):
    import torch
    import torch.distributed as dist
    from nv_embedding_cache_b200 import workloads
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    fn = {"c3": workloads.run_c3, "c4a": workloads.run_c4a, "c4b": workloads.run_c4b,
          "c5": workloads.run_c5, "published": workloads.run_published_gpulayer}[args.workload]
    steps = min(args.steps, 50)
    kw = {}
    if args.rows > 0:   # smaller table for profiling runs (the configuration's size is the default)
        kw["rows_per_rank" if args.workload == "c5" else "rows"] = args.rows
    if args.workload in ("c3", "c4a", "c4b") and world == 1:
        kw["ref_gpu"] = load_reference_gpu()
    res = fn(str(ROOT), steps=steps, warmup=args.warmup, **kw)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the device-resident leg directly instead of replaying CUDA graphs")
    ap.add_argument("--workload", choices=["c2", "c3", "c4a", "c4b", "c5", "published"], default="c2",
                    help="c2 is the headline benchmark; the others print one JSON line for that "
                         "configuration (see nv_embedding_cache_b200/workloads.py)")
    ap.add_argument("--rows", type=int, default=0,
                    help="table rows for --workload runs (0 = the configuration's own size)")
    ap.add_argument("--tables", type=int, default=NUM_TABLES,
                    help="tables per GPU (profiling runs use fewer; the benchmark config is 8)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    globals()["NUM_TABLES"] = max(1, min(8, args.tables))
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload != "c2":
        run_other_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
