#!/usr/bin/env python
"""Benchmark of the embedding lookup hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (BASELINE config "GPULayer, fully HBM-resident"): 8 independent tables of
4,000,000 rows x 128 fp16 (N(0, 0.02)); per table 65,536 bags of 1..32 int64 keys, Zipf(1.1) over a
permuted row order, CSR offsets, mean pooling accumulated in fp32, output [65536,128] fp16.  One
*step* is one pooled lookup of every table (8 launches of the fused gather+pool kernel).  Tables and
key batches are seeded synthetic data.  With N > 1 every rank serves its own 8 tables (independent
tables: no data-path collective, weak scaling).

The JSON line (rank 0) also carries, measured in the same run:
  sharded    the NVLink-sharded table (250M x W rows x 64 fp16, 32 GB per GPU) at this world size: the
             peer form, the peer form behind the replicated hot-row table and the exchange form, each
             with keys/s, NVLink GB/s per rank, a parity flag against the oracle and its clock record
  workloads  (one GPU) int8 dequantise + pool, gradient de-duplication + update, and the cached gather
             from a 25.6 GB host table, each with roofline, clocks, end-to-end and CPU figures
  low_reuse  (one GPU) the headline kernel on key streams that really reach HBM
  copy_probe (several GPUs) what the host side gives all ranks' pinned copies at once
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
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
REPEATS = 5              # timed regions per leg; the median one is reported
METRIC = "embedding keys/sec (find-and-combine)"
WORKLOAD = "C2 GPULayer HBM-resident: 8 tables x 4M x 128 fp16, 65536 CSR bags len U[1,32], Zipf(1.1), mean pool fp32 acc"


def bench_config(world: int) -> dict:
    """The workload both arms measure (identical keys and values in both JSON lines)."""
    return {"workload": WORKLOAD, "tables_per_gpu": NUM_TABLES, "rows_per_table": NUM_ROWS,
            "bags_per_table": NUM_BAGS, "key_batches_cycled": NUM_BATCHES,
            "l2": "inputs larger than L2 (8.2 GB of tables, 4 key batches cycled)",
            "parallelism": f"replicas x{world} (independent tables, no collective)"}


def make_batch(table_idx: int, batch_idx: int, rank: int, perm: np.ndarray, alpha: float = ALPHA,
               num_rows: int = NUM_ROWS):
    from nv_embedding_cache_b200 import datagen as dg
    seed = 1000 + 200 + 10 * table_idx + batch_idx + 1000 * rank
    _, offsets = dg.csr_bags(NUM_BAGS, 1, 32, seed)
    if alpha is None:
        keys = dg.uniform_keys(int(offsets[-1]), num_rows, seed + 5000)
    else:
        keys = dg.zipf_keys(int(offsets[-1]), num_rows, alpha, seed + 5000, perm)
    return keys, offsets


def algorithmic_bytes(num_keys: int) -> int:
    """Bytes one pooled lookup must move: keys + rows read, offsets read, pooled rows written."""
    return num_keys * (8 + ROW_BYTES) + (NUM_BAGS + 1) * 8 + NUM_BAGS * ROW_BYTES


def load_reference_gpu():
    """The unmodified reference GPU code built into oracle/_ref (a baseline timed beside this
    library's kernels, never on their path); None when the library was not built."""
    try:
        from oracle.pyoracle import ReferenceGpu
        return ReferenceGpu()
    except (FileNotFoundError, OSError):
        return None


# ---- reference arm: the reference's own CPU path on this box's host cores ----------------------------
def run_reference_arm(args):
    """--impl reference: HostEmbeddingLayer over a LinearHostTable (the unmodified reference sources
    built into oracle/_ref, with the SIMD flags its own build picks on this host), one table's pooled
    lookup per step, default thread pool."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from nv_embedding_cache_b200 import datagen as dg
    from oracle.pyoracle import Reference
    perm = dg.permutation(NUM_ROWS)
    table = dg.normal_table(NUM_ROWS, WIDTH, 0.02, 20, np.float16)
    batches = [make_batch(0, b, 0, perm) for b in range(NUM_BATCHES)]
    ref = Reference(for_timing=True)
    layer = ref.layer(table.view(np.uint8).reshape(NUM_ROWS, ROW_BYTES), "f16")
    workers = layer.num_workers
    out = np.zeros((NUM_BAGS, WIDTH), dtype=np.float16)

    def step(i):
        keys, offsets = batches[i % NUM_BATCHES]
        layer.lookup_pooled(keys, "mean", WIDTH, offsets=offsets, out_dtype="f16", out=out)
        return keys.size

    for i in range(max(args.warmup, 1)):
        step(i)
    times, nkeys = [], 0
    t_end = time.perf_counter() + args.cpu_seconds
    i = 0
    while i < args.steps or (args.cpu_seconds > 0 and time.perf_counter() < t_end and i < 400):
        t0 = time.perf_counter()
        nkeys += step(i)
        times.append(time.perf_counter() - t0)
        i += 1
    layer.close()
    dt = float(sum(times))
    value = nkeys / dt
    sample = (f"each step = one table's pooled lookup ({batches[0][0].size} keys, 65536 bags) of the 8-table "
              f"workload; {len(times)} steps, median {np.median(times) * 1e3:.1f} ms, mean {np.mean(times) * 1e3:.1f} ms "
              f"per step; reference CPU sources built with {ref.simd}")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "keys/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / max(1, len(times)), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": bench_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "keys/s", "cores": int(workers),
                         "kind": "reference", "sample": sample, "host_cpus": os.cpu_count(),
                         "median_keys_per_s": batches[0][0].size / float(np.median(times))},
        "e2e": {"value": value, "unit": "keys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def cpu_baseline_in_child(seconds: float):
    """The reference arm in a process of its own, before this process touches the GPU: the same code
    and the same conditions as `--impl reference`, so the two figures of one box agree."""
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "5", "--warmup", "2",
           "--cpu-seconds", str(seconds)]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    for line in reversed(res.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)["cpu_baseline"]
    raise RuntimeError(f"reference arm gave no line: {res.stderr[-400:]}")


# ---- this library --------------------------------------------------------------------------------------
def run_ours(args):
    skip = set(filter(None, args.skip.split(",")))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    # the CPU baseline first, in a child process, while this process holds no GPU memory, no pinned
    # buffers and no sampler thread
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu_baseline = cpu_baseline_in_child(args.cpu_seconds)
        except Exception as e:  # the checker library is absent: report, do not fake
            cpu_baseline = {"value": None, "unit": "keys/s", "cores": 0, "kind": "reference",
                            "sample": f"unavailable: {e}"}

    import torch
    import torch.distributed as dist
    import bench_workloads as bw
    from nv_embedding_cache_b200 import datagen as dg
    from nv_embedding_cache_b200.layers import GPUEmbeddingLayer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the lookup path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

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
        for t in range(NUM_TABLES):
            k, o = dev_batches[t][i % NUM_BATCHES]
            layers[t].lookup_pooled(ctxs[t], k.numel(), k, dev_out[t], ROW_BYTES, "mean", "float16",
                                    csr_offsets=o, num_csr_offsets=o.numel())

    def step_host(i):
        for t in range(NUM_TABLES):
            k, o = pin_batches[t][i % NUM_BATCHES]
            layers[t].lookup_pooled(ctxs_e2e[t], k.numel(), k, pin_out[t], ROW_BYTES, "mean",
                                    "float16", csr_offsets=o, num_csr_offsets=o.numel())

    keys_of_step = [sum(dev_batches[t][b][0].numel() for t in range(NUM_TABLES)) for b in range(NUM_BATCHES)]
    h2d_of_step = [sum((k.numel() + o.numel()) * 8 for k, o in (pin_batches[t][b] for t in range(NUM_TABLES)))
                   for b in range(NUM_BATCHES)]

    # One step of the device-resident leg is eight short launches issued from Python, about as long
    # on the host as on the GPU.  Each of the four cycled steps is therefore captured once as a CUDA
    # graph and replayed (same kernels, same arguments); --no-graph, or a capture that fails, keeps
    # the direct launches.  The capture runs BEFORE the process group of a multi-rank run exists, so
    # every rank captures exactly as a single-rank run does, with no communicator and none of its
    # threads in the process, and every world size measures the same launch mode.
    graphs = []
    if not args.no_graph:
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
    torch.cuda.synchronize()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def step_replay(i):
        graphs[i % NUM_BATCHES].replay()

    def region(fn, steps, fan_out):
        """One timed region of exactly `steps` steps: barrier + synchronize on both sides, CUDA events
        on the launching stream, the maximum over the ranks."""
        bw.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if fan_out:
            for ts in table_streams:
                ts.wait_event(e0)
        for i in range(steps):
            fn(i)
        if fan_out:
            for ts in table_streams:
                ev = torch.cuda.Event()
                ev.record(ts)
                stream.wait_event(ev)
        e1.record(stream)
        bw.barrier()
        return bw.reduce_max(e0.elapsed_time(e1))

    # steps cycle the four batches: a region of K steps looks up sum over i < K of keys_of_step[i % 4]
    keys_region = sum(keys_of_step[i % NUM_BATCHES] for i in range(args.steps))
    h2d_region = sum(h2d_of_step[i % NUM_BATCHES] for i in range(args.steps))
    with torch.cuda.stream(stream):
        dev_fn = step_replay if graphs else step_device
        for i in range(args.warmup):
            dev_fn(i)
        with bw.ClockSampler.for_current_device(period_s=0.004) as clk:
            dev_regions = [region(dev_fn, args.steps, False) for _ in range(REPEATS)]
            clk.sample_now()
        clocks = clk.summary()
        for i in range(args.warmup):
            step_host(i)
        e2e_regions = [region(step_host, args.steps, True) for _ in range(3)]
    ms_dev = float(np.median(dev_regions))
    ms_e2e = float(np.median(e2e_regions))
    value = bw.reduce_sum(keys_region) / (ms_dev * 1e-3)
    e2e_value = bw.reduce_sum(keys_region) / (ms_e2e * 1e-3)

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

    # ---- roofline of the dominant kernel (this rank): algorithmic bytes per launch / mean launch time
    launches = args.steps * NUM_TABLES
    mean_launch_s = ms_dev * 1e-3 / launches
    alg_bytes = algorithmic_bytes(keys_region // launches)
    peak, peak_kind = bw.hbm_peak()
    achieved = alg_bytes / mean_launch_s / 1e9
    roofline = {"bound": "hbm", "kernel": "pool_dense_kernel<F16,GROUP=16,U=8>",
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": achieved / peak, "traffic": None,
                "algorithmic_bytes_per_launch": alg_bytes, "mean_launch_us": mean_launch_s * 1e6,
                # beside the measured copy rate, the data-sheet figure of the part (8 TB/s HBM3e)
                "frac_of_nominal_8tbs": achieved / 8000.0}
    traffic_file = ROOT / "profiles" / "lookup_pool_f16_c2.traffic.json"
    if traffic_file.exists():
        roofline["traffic"] = json.loads(traffic_file.read_text()).get("dram_bytes_per_launch")
        if roofline["traffic"]:
            roofline["frac_on_dram_bytes"] = roofline["traffic"] / mean_launch_s / 1e9 / peak

    out = {
        "metric": METRIC, "value": value, "unit": "keys/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": bench_config(world),
        "launch": "CUDA graph of one step (8 kernels), replayed" if graphs else "direct launches",
        "keys_per_step_per_gpu": keys_region // args.steps,
        "timing": {"regions": REPEATS, "reported": "median region; every region is exactly `steps` steps between "
                   "barrier + synchronize, CUDA events on the launching stream, max over ranks",
                   "region_ms": [round(r, 4) for r in dev_regions], "e2e_region_ms": [round(r, 4) for r in e2e_regions]},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "keys/s",
                "h2d_bytes_per_step": h2d_region // args.steps,
                "d2h_bytes_per_step": NUM_TABLES * NUM_BAGS * ROW_BYTES,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": (REPEATS + 3) * launches,
        "roofline": roofline,
        "algo_bw_gib_s": value * ROW_BYTES / 2**30,
        "per_launch": per_launch,
    }
    if cpu_baseline is not None:
        out["cpu_baseline"] = cpu_baseline

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

    # ---- the same kernel on key streams that reach HBM (one GPU): uniform keys over a 4M-row table,
    # and Zipf(1.1) over a table ten times larger
    if world == 1 and "low_reuse" not in skip:
        with torch.cuda.stream(stream):
            out["low_reuse"] = low_reuse_runs(args, torch, bw, dg, GPUEmbeddingLayer, tables[0], dev, stream)

    for c in ctxs + ctxs_e2e:
        c.wait()
        c.destroy()
    for layer in layers:
        layer.destroy()
    del tables, dev_batches, pin_batches, dev_out, pin_out, graphs
    torch.cuda.empty_cache()

    if world > 1 and "copy_probe" not in skip:
        out["copy_probe"] = bw.copy_probe()
    if "sharded" not in skip:
        kw = {"rows_per_rank": args.shard_rows} if args.shard_rows > 0 else {}
        out["sharded"] = bw.sharded_record(steps=args.steps, warmup=args.warmup, repeats=REPEATS, **kw)
    if world == 1 and "workloads" not in skip:
        w = {}
        for name, fn in (("c4a", bw.record_c4a), ("c4b", bw.record_c4b), ("c3", bw.record_c3)):
            if name in skip:
                continue
            try:
                w[name] = fn()
            except Exception as e:  # noqa: BLE001 - one configuration must not take the line down
                w[name] = {"error": f"{type(e).__name__}: {e}"}
        out["workloads"] = w

    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def low_reuse_runs(args, torch, bw, dg, GPUEmbeddingLayer, table0, dev, stream):
    """pool_dense_kernel on the headline shape when few rows repeat: DRAM traffic then approaches the
    algorithmic bytes, and the fraction of the HBM peak is a statement about HBM."""
    res = {}
    peak, kind = bw.hbm_peak()
    cases = [("uniform_4M", table0, NUM_ROWS, None)]
    big_rows = args.low_reuse_rows if args.low_reuse_rows > 0 else 40_000_000
    try:
        big = torch.empty((big_rows, WIDTH), dtype=torch.float16, device=dev)
        gen = torch.Generator(device=dev)
        gen.manual_seed(77)
        chunk = 1 << 22
        for r0 in range(0, big_rows, chunk):
            r1 = min(big_rows, r0 + chunk)
            big[r0:r1] = (torch.randn((r1 - r0, WIDTH), generator=gen, device=dev) * 0.02).half()
        tag = f"{big_rows // 1_000_000}M"
        cases.append((f"zipf1.1_{tag}", big, big_rows, ALPHA))
        cases.append((f"uniform_{tag}", big, big_rows, None))
    except Exception as e:  # noqa: BLE001
        res["zipf1.1_40M"] = {"error": str(e)}
    for name, table, rows, alpha in cases:
        batches = []
        for b in range(NUM_BATCHES):
            # perm None: the Zipf ranks go through the table-free affine permutation of the row ids
            k, o = make_batch(0, b, 7, None, alpha=alpha, num_rows=rows)
            batches.append((torch.from_numpy(k).to(dev), torch.from_numpy(o).to(dev)))
        layer = GPUEmbeddingLayer(table, rows, ROW_BYTES, "float16", device_id=dev.index, layer_name=name)
        ctx = layer.create_execution_context(stream.cuda_stream, stream.cuda_stream)
        outb = torch.empty((NUM_BAGS, WIDTH), dtype=torch.float16, device=dev)

        def step(i):
            k, o = batches[i % NUM_BATCHES]
            layer.lookup_pooled(ctx, k.numel(), k, outb, ROW_BYTES, "mean", "float16", csr_offsets=o,
                                num_csr_offsets=o.numel())
        ms, regions = bw.timed_repeats(stream, step, args.steps * NUM_TABLES, args.warmup, REPEATS)
        sec = ms * 1e-3 / (args.steps * NUM_TABLES)
        nk = float(np.mean([k.numel() for k, _ in batches]))
        alg = algorithmic_bytes(int(nk))
        # rows that are read once per launch come from DRAM: distinct keys * row bytes (+ keys, offsets, output)
        distinct = float(np.mean([torch.unique(k).numel() for k, _ in batches]))
        dram_est = distinct * ROW_BYTES + nk * 8 + (NUM_BAGS + 1) * 8 + NUM_BAGS * ROW_BYTES
        entry = {"keys_per_s": nk / sec, "us_per_launch": sec * 1e6, "distinct_keys_per_launch": distinct,
                 "algorithmic_gbs": alg / sec / 1e9, "frac": alg / sec / 1e9 / peak,
                 "dram_bytes_estimate": int(dram_est), "frac_on_dram_estimate": dram_est / sec / 1e9 / peak,
                 "peak_kind": kind, "region_ms": [round(r, 4) for r in regions]}
        tf = ROOT / "profiles" / f"pool_dense_f16_{name}.traffic.json"
        if tf.exists():
            entry["traffic"] = json.loads(tf.read_text()).get("dram_bytes_per_launch")
            if entry["traffic"]:
                entry["frac_on_dram_bytes"] = entry["traffic"] / sec / 1e9 / peak
        res[name] = entry
        ctx.wait()
        ctx.destroy()
        layer.destroy()
    return res


def run_other_workload(args):
    import torch
    import torch.distributed as dist
    import bench_workloads as workloads
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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--cpu-seconds", type=float, default=None,
                    help="time budget of the CPU baseline (ours: 12 s in a child process; reference arm: "
                         "0 = exactly --steps steps)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the device-resident leg directly instead of replaying CUDA graphs")
    ap.add_argument("--workload", choices=["c2", "c3", "c4a", "c4b", "c5", "published"], default="c2",
                    help="c2 is the headline benchmark; the others print one JSON line for that "
                         "configuration (see bench_workloads.py)")
    ap.add_argument("--rows", type=int, default=0,
                    help="table rows for --workload runs (0 = the configuration's own size)")
    ap.add_argument("--shard-rows", type=int, default=0,
                    help="rows per rank of the sharded record (0 = 250,000,000; profiling runs use fewer)")
    ap.add_argument("--low-reuse-rows", type=int, default=0,
                    help="rows of the larger table of the low-reuse runs (0 = 40,000,000; profiler captures use fewer)")
    ap.add_argument("--skip", default="",
                    help="comma list of parts to leave out of the line: sharded, workloads, c4a, c4b, c3, "
                         "low_reuse, copy_probe")
    ap.add_argument("--tables", type=int, default=NUM_TABLES,
                    help="tables per GPU (profiling runs use fewer; the benchmark config is 8)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    if args.cpu_seconds is None:
        args.cpu_seconds = 12.0 if args.impl == "ours" else 0.0
    globals()["NUM_TABLES"] = max(1, min(8, args.tables))
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload != "c2":
        run_other_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
