"""Threading contract of the layer API (reference docs/advanced.md:3-11, include/nve_c_api.h:516-526):
a context is used by one thread at a time; different contexts of one layer may run lookups
concurrently from different threads while another thread modifies the cache."""
import threading

import numpy as np
import pytest

from nv_embedding_cache_b200 import datagen as dg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kernel_mode", [0, 2, 3], ids=["fused", "sort_gather", "pipeline"])
def test_concurrent_lookups_and_inserts(torch_cuda, kernel_mode):
    """Every lookup schedule: the sort-gather and pipeline schedules spread one lookup over several
    kernels (the pipeline one over auxiliary streams and host threads as well), so an insert that
    lands between them must not change what the lookup copies."""
    torch = torch_cuda
    from nv_embedding_cache_b200.layers import GpuTable, LinearUVMEmbeddingLayer
    rows, dim = 50_000, 64
    table = dg.normal_table(rows, dim, 0.02, 1, np.float16)
    backing = torch.from_numpy(table).pin_memory()
    tb = table.view(np.uint8).reshape(rows, -1)
    gt = GpuTable((8000 // 8) * (64 + 8 * dim * 2 + 32), dim * 2, "float16", uvm_table=backing, uvm_num_rows=rows,
                  kernel_mode_type=kernel_mode)
    layer = LinearUVMEmbeddingLayer(gt)
    perm = dg.permutation(rows)
    errors = []

    def reader(tid):
        try:
            stream = torch.cuda.Stream()
            ctx = layer.create_execution_context(stream.cuda_stream, stream.cuda_stream)
            for it in range(40):
                keys = dg.zipf_keys(3000, rows, 1.2, 1000 * tid + it, perm)
                out = np.zeros((keys.size, dim), np.float16)
                layer.lookup(ctx, keys.size, keys, out, dim * 2)
                ctx.wait()
                if not np.array_equal(out, table[keys]):
                    errors.append(f"reader {tid} iteration {it}: wrong rows")
                    break
                _, offs = dg.csr_bags(200, 1, 12, 77 + it)
                pk = dg.zipf_keys(int(offs[-1]), rows, 1.2, 5000 * tid + it, perm)
                pooled = np.zeros((200, dim), np.float16)
                layer.lookup_pooled(ctx, pk.size, pk, pooled, dim * 2, "sum", "float16",
                                    csr_offsets=offs, num_csr_offsets=offs.size)
                ctx.wait()
                want = np.stack([table[pk[offs[b]:offs[b + 1]]].astype(np.float32).sum(0) for b in range(200)])
                if np.max(np.abs(pooled.astype(np.float32) - want)) > 2e-3:
                    errors.append(f"reader {tid} iteration {it}: wrong pooled rows")
                    break
            ctx.destroy()
        except Exception as e:  # noqa: BLE001 - reported to the main thread
            errors.append(f"reader {tid}: {e!r}")

    def writer():
        try:
            stream = torch.cuda.Stream()
            ctx = layer.create_execution_context(stream.cuda_stream, stream.cuda_stream)
            for it in range(25):
                keys = dg.zipf_keys(2000, rows, 1.2, 9000 + it, perm)
                layer.insert(ctx, keys.size, keys, dim * 2, dim * 2, tb[keys])
                if it % 5 == 4:
                    gone = np.unique(keys)[:300]
                    layer.erase(ctx, gone.size, gone)
                ctx.wait()
            ctx.destroy()
        except Exception as e:  # noqa: BLE001
            errors.append(f"writer: {e!r}")

    threads = [threading.Thread(target=reader, args=(t,)) for t in range(4)] + [threading.Thread(target=writer)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not any(t.is_alive() for t in threads), "a thread did not finish"
    assert not errors, errors
    layer.destroy()
    gt.destroy()
