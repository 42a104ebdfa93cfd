"""The compiled torch ops (libnve_b200_torch_ops.so), the layer registry behind them
(nve_b200_registry_*), and saving / reloading models through nv_embedding_cache_b200.export.

Without a GPU: the op library loads, carries the reference's schemas
(python/pynve/torch_bindings/torch_binding.cpp:86-91), infers shapes for fake tensors, refuses host
tensors, and the registry's argument errors come back as statuses.  With a GPU: the ops give the
rows the plain path gives, layers train beside torch.nn through them, a model goes through
export -> load in a child interpreter (as a deployment would) and through save -> load with shared
storage, and unknown or stale markers are reported, not followed.
"""
import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _ops():
    import torch
    from nv_embedding_cache_b200 import torch_layers as L
    assert L.HAS_TORCH_OPS, "libnve_b200_torch_ops.so is missing: python -m nv_embedding_cache_b200.build"
    return torch, L


def test_op_library_defines_the_reference_schemas():
    torch, _ = _ops()
    assert str(torch.ops.nve_ops.embedding_lookup.default._schema) == \
        "nve_ops::embedding_lookup(Tensor marker, Tensor keys, int embedding_size, int dtype) -> Tensor"
    assert str(torch.ops.nve_ops.embedding_lookup_with_pooling.default._schema) == \
        ("nve_ops::embedding_lookup_with_pooling(Tensor marker, Tensor keys, Tensor offsets, Tensor? weights, "
         "int pooling_type, int embedding_size, int dtype) -> Tensor")


def test_shapes_are_inferred_without_a_layer():
    torch, L = _ops()
    from nv_embedding_cache_b200 import pynve
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        marker = torch.zeros(1, dtype=torch.int64)
        keys = torch.zeros((3, 4), dtype=torch.int64)
        offsets = torch.zeros(7, dtype=torch.int64)
        a = torch.ops.nve_ops.embedding_lookup(marker, keys, 24, int(pynve.DataType_t.Float16))
        b = torch.ops.nve_ops.embedding_lookup_with_pooling(marker, keys.reshape(-1), offsets, None,
                                                            int(pynve.PoolingType_t.Sum), 24,
                                                            int(pynve.DataType_t.Float32))
    assert tuple(a.shape) == (12, 24) and a.dtype == torch.float16
    assert tuple(b.shape) == (6, 24) and b.dtype == torch.float32


def test_host_tensors_are_refused():
    torch, _ = _ops()
    with pytest.raises(RuntimeError, match="keys are on the host"):
        torch.ops.nve_ops.embedding_lookup(torch.zeros(1, dtype=torch.int64), torch.arange(4), 8, 1)


def test_ops_are_traced_by_torch_export():
    """Tracing needs no layer and no GPU: shapes come from the registered shape functions, the marker
    becomes a constant of the graph, and the saved program comes back with that constant as a buffer
    a loader can re-point."""
    import io
    torch, L = _ops()

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("marker_tensor", torch.tensor([7]), persistent=False)
            self.head = torch.nn.Linear(8, 2)

        def forward(self, keys, offsets):
            L._check_forward_inputs(keys, offsets)
            rows = L.MarkerLookupOp.apply(self.marker_tensor, keys, None, 8, 1)
            bags = L.MarkerPooledLookupOp.apply(self.marker_tensor, keys, None, offsets, None, 1, 8, 1)
            return self.head(rows).sum() + self.head(bags).sum()

    n, b = torch.export.Dim("n", min=2, max=1000), torch.export.Dim("b", min=3, max=1000)
    program = torch.export.export(Net(), (torch.arange(6), torch.arange(0, 7, 2)),
                                  dynamic_shapes={"keys": {0: n}, "offsets": {0: b}})
    targets = [str(node.target) for node in program.graph.nodes if node.op == "call_function"]
    assert "nve_ops.embedding_lookup.default" in targets
    assert "nve_ops.embedding_lookup_with_pooling.default" in targets
    buf = io.BytesIO()
    torch.export.save(program, buf)
    buf.seek(0)
    module = torch.export.load(buf).module()
    assert dict(module.named_buffers())["marker_tensor"].tolist() == [7]


def test_registry_argument_errors(capi):
    lib = capi.lib
    assert lib.nve_b200_registry_size() >= 0
    assert lib.nve_b200_registry_register(None, 1, 8, capi.DTYPE_FLOAT32, 0) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert lib.nve_b200_registry_register(1, None, 8, capi.DTYPE_FLOAT32, 0) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert lib.nve_b200_registry_register(1, 1, 0, capi.DTYPE_FLOAT32, 0) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert lib.nve_b200_registry_register(1, 1, 8, capi.DTYPE_UNKNOWN, 0) == capi.NVE_ERROR_INVALID_ARGUMENT
    dim = C.c_int64()
    assert lib.nve_b200_registry_describe(0x1234, C.byref(dim), None, None) == capi.NVE_ERROR_INVALID_ARGUMENT
    msg = C.c_char_p()
    lib.nve_get_last_error(C.byref(msg))
    assert b"no layer is registered" in msg.value
    assert lib.nve_b200_registry_lookup(0x1234, 0, None, None, None) == capi.NVE_ERROR_INVALID_ARGUMENT
    assert lib.nve_b200_registry_unregister(0x1234) == capi.NVE_SUCCESS      # unknown markers are ignored


def test_config_and_block_names_for_metadata():
    from nv_embedding_cache_b200 import pynve
    cfg = pynve.EmbedLayerConfig()
    cfg.kernel_mode, cfg.default_row_index = 2, 7
    doc = json.loads(cfg.to_json())
    assert doc["kernel_mode"] == 2 and doc["default_row_index"] == 7 and doc["default_embedding"] == []
    assert set(doc) == {"logging_interval", "kernel_mode", "kernel_mode_value_1", "kernel_mode_value_2",
                        "max_modify_size", "default_row_index", "default_embedding"}
    assert pynve.MemBlockType.Managed.name == "Managed" and pynve.MemBlockType.User == "User"
    assert pynve.resolve_memblock_devices(pynve.MemBlockType.Managed, 3) == [3]
    assert pynve.resolve_memblock_devices(pynve.MemBlockType.NVL, 0, [2, 5]) == [2, 5]


def test_metadata_rules_need_no_gpu(tmp_path):
    """Which block replaces a caller-owned one, and what a loader refuses before it builds anything."""
    import torch
    from nv_embedding_cache_b200 import export as E, torch_layers as L
    G, U = L.LayerType.GPULayer, L.LayerType.LinearUVM
    assert E._block_kind_for({G}) == "Linear" and E._block_kind_for({G, U}) == "Linear"
    assert E._block_kind_for({U}) == "Managed"
    with pytest.raises(ValueError):
        E._block_kind_for({L.LayerType.HostLayer})
    where = torch.device("cuda", 0)
    (tmp_path / "metadata.json").write_text(json.dumps({"version": 3, "resources": {}, "layers": []}))
    with pytest.raises(RuntimeError, match="schema version 3"):
        E.load_nve_layers(str(tmp_path), device=where)
    entry = {"id": 1, "module_path": "emb", "num_embeddings": 10, "embedding_size": 4, "dtype": "float32",
             "layer_type": "Hierarchical", "gpu_cache_size": 0, "optimize_for_training": False}
    (tmp_path / "metadata.json").write_text(json.dumps({"version": 2, "resources": {}, "layers": [entry]}))
    with pytest.raises(NotImplementedError, match="Hierarchical"):
        E.load_nve_layers(str(tmp_path), device=where)
    entry["layer_type"] = "GPULayer"
    (tmp_path / "metadata.json").write_text(json.dumps({"version": 2, "resources": {}, "layers": [entry]}))
    with pytest.raises(ValueError, match="names no storage block"):
        E.load_nve_layers(str(tmp_path), device=where)
    entry["storage_ref"] = "mb-1"
    (tmp_path / "metadata.json").write_text(json.dumps({"version": 2, "resources": {"memblocks": {}},
                                                        "layers": [entry]}))
    with pytest.raises(ValueError, match="not among resources"):
        E.load_nve_layers(str(tmp_path), device=where)
    with pytest.raises(ValueError, match="layers of this library live on a cuda device"):
        E.load_nve_layers(str(tmp_path), device=torch.device("cpu"))


def _table(torch, rows, dim, dtype):
    g = torch.Generator(device="cuda").manual_seed(rows + dim)
    return (torch.randint(-64, 65, (rows, dim), generator=g, device="cuda") / 32.0).to(dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("layer_type", ["GPULayer", "LinearUVM"])
@pytest.mark.parametrize("dtype_name", ["float32", "float16"])
def test_ops_give_the_rows_of_the_plain_path(torch_cuda, layer_type, dtype_name):
    torch, L = _ops()
    from nv_embedding_cache_b200 import pynve
    dtype = getattr(torch, dtype_name)
    rows, dim = 3000, 48
    w = _table(torch, rows, dim, dtype)
    kw = dict(gpu_cache_size=1 << 20) if layer_type == "LinearUVM" else {}
    before = pynve.capi.lib.nve_b200_registry_size()
    layer = L.NVEmbeddingBag(rows, dim, dtype, getattr(L.LayerType, layer_type), "mean", weight_init=w, **kw)
    assert pynve.capi.lib.nve_b200_registry_size() == before + 1
    rng = np.random.default_rng(1)
    keys = torch.from_numpy(rng.integers(0, rows, 640)).cuda()
    cuts = np.sort(rng.integers(0, 641, 127))          # 128 bags, some of them empty
    offsets = torch.from_numpy(np.concatenate([[0], cuts, [640]])).cuda()
    # the dense layer wants weights of the rows' own type (a rule of the reference layer)
    weights = torch.from_numpy(rng.integers(1, 5, 640).astype(np.float32)).cuda().to(dtype)
    marker, tag = layer.marker_tensor, layer.dtype_tag

    got = torch.ops.nve_ops.embedding_lookup(marker, keys, dim, tag)
    assert torch.equal(got, w[keys])
    for pool, wts in ((pynve.PoolingType_t.Sum, None), (pynve.PoolingType_t.Mean, None),
                      (pynve.PoolingType_t.WeightedSum, weights), (pynve.PoolingType_t.WeightedMean, weights)):
        got = torch.ops.nve_ops.embedding_lookup_with_pooling(marker, keys, offsets, wts, int(pool), dim, tag)
        want = torch.empty_like(got)
        layer.emb_layer.lookup_with_pooling(keys.numel(), keys.data_ptr(), want.data_ptr(), int(pool),
                                            offsets.numel(), offsets.data_ptr(),
                                            tag if wts is not None else int(pynve.DataType_t.Float32),
                                            wts.data_ptr() if wts is not None else 0,
                                            torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(got, want), pool
    # a side stream gets its own execution context inside the registry
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = torch.ops.nve_ops.embedding_lookup(marker, keys, dim, tag)
    side.synchronize()
    assert torch.equal(got, w[keys])
    # arguments baked into a graph that do not fit the layer are refused
    with pytest.raises(RuntimeError, match="embedding_size"):
        torch.ops.nve_ops.embedding_lookup(marker, keys, dim + 1, tag)
    with pytest.raises(RuntimeError, match="data type"):
        torch.ops.nve_ops.embedding_lookup(marker, keys, dim, 1 if tag != 1 else 3)
    with pytest.raises(RuntimeError, match="int64"):
        torch.ops.nve_ops.embedding_lookup(marker, keys.int(), dim, tag)
    with pytest.raises(RuntimeError, match="one element per key"):
        torch.ops.nve_ops.embedding_lookup_with_pooling(marker, keys, offsets, weights[:-1], 3, dim, tag)
    stale = marker.clone()
    with pytest.raises(RuntimeError, match="no layer is registered"):
        torch.ops.nve_ops.embedding_lookup(stale, keys, dim, tag)
    del layer
    import gc
    gc.collect()
    assert pynve.capi.lib.nve_b200_registry_size() == before


@pytest.mark.gpu
@pytest.mark.parametrize("layer_type", ["GPULayer", "LinearUVM"])
def test_layers_train_beside_torch_through_the_ops(torch_cuda, layer_type):
    torch, L = _ops()
    rows, dim = 2000, 32
    w0 = _table(torch, rows, dim, torch.float32)
    kind = getattr(L.LayerType, layer_type)
    kw = dict(gpu_cache_size=1 << 20) if layer_type == "LinearUVM" else {}
    emb = L.NVEmbedding(rows, dim, torch.float32, kind, weight_init=w0.clone(), **kw)
    bag = L.NVEmbeddingBag(rows, dim, torch.float32, kind, "sum", weight_init=w0.clone(), **kw)
    t_emb = torch.nn.Embedding(rows, dim, sparse=True, device="cuda")
    t_bag = torch.nn.EmbeddingBag(rows, dim, mode="sum", sparse=True, include_last_offset=True, device="cuda")
    with torch.no_grad():
        t_emb.weight.copy_(w0)
        t_bag.weight.copy_(w0)
    opts = [torch.optim.SGD(m.parameters(), lr=0.5) for m in (emb, bag, t_emb, t_bag)]
    rng = np.random.default_rng(3)
    for _ in range(4):
        keys = torch.from_numpy(rng.integers(0, rows, 256)).cuda()
        offs = torch.arange(0, 257, 4, device="cuda")
        outs = [emb(keys), bag(keys, offs), t_emb(keys), t_bag(keys, offs)]
        assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
        for o, opt in zip(outs, opts):
            opt.zero_grad()
            (o * 0.25).sum().backward()
            opt.step()
    torch.cuda.synchronize()
    probe = torch.arange(rows, device="cuda")
    assert torch.equal(emb(probe), t_emb(probe))
    frozen = L.NVEmbedding(rows, dim, torch.float32, kind, weight_init=w0, optimize_for_training=False, **kw)
    out = frozen(probe[:8])
    assert not out.requires_grad


MODEL = """
import torch
from nv_embedding_cache_b200 import torch_layers as L

class Model(torch.nn.Module):
    def __init__(self, w_a=None, w_b=None):
        super().__init__()
        self.emb = L.NVEmbedding(500, 16, torch.float32, L.LayerType.GPULayer, optimize_for_training=False,
                                 weight_init=w_a, id=11)
        self.bag = L.NVEmbeddingBag(800, 16, torch.float16, L.LayerType.LinearUVM, "sum", gpu_cache_size=1 << 20,
                                    optimize_for_training=False, weight_init=w_b, id=12)
        self.head = torch.nn.Linear(16, 4)

    def forward(self, keys, bag_keys, offsets):
        return self.head(self.emb(keys) + self.bag(bag_keys, offsets).float().repeat_interleave(4, 0))
"""


@pytest.mark.gpu
def test_export_then_load_in_another_process(torch_cuda, tmp_path):
    """export writes metadata, tables and the traced program; a fresh interpreter that never saw the
    model class loads them and gets the same outputs, also for a batch of another size."""
    torch, L = _ops()
    from nv_embedding_cache_b200 import export as E
    scope = {}
    exec(MODEL, scope)
    w_a = _table(torch, 500, 16, torch.float32)
    w_b = _table(torch, 800, 16, torch.float16)
    model = scope["Model"](w_a, w_b).cuda().eval()
    torch.manual_seed(0)
    keys = torch.randint(0, 500, (64,), device="cuda")
    bag_keys = torch.randint(0, 800, (48,), device="cuda")
    offsets = torch.arange(0, 49, 3, device="cuda")
    want = model(keys, bag_keys, offsets)
    keys2, bag_keys2, offsets2 = keys[:32].contiguous(), bag_keys[:24].contiguous(), offsets[:9].contiguous()
    want2 = model(keys2, bag_keys2, offsets2)
    batch = torch.export.Dim("batch", min=2, max=4096)
    bagged = torch.export.Dim("bagged", min=2, max=1 << 20)
    E.export(model, (keys, bag_keys, offsets), str(tmp_path),
             dynamic_shapes={"keys": {0: 4 * batch}, "bag_keys": {0: bagged}, "offsets": {0: batch + 1}})
    doc = json.loads((tmp_path / "metadata.json").read_text())
    assert doc["version"] == 2 and [e["module_path"] for e in doc["layers"]] == ["emb", "bag"]
    kinds = {doc["resources"]["memblocks"][e["storage_ref"]]["type"] for e in doc["layers"]}
    assert kinds == {"Linear", "Managed"}       # the caller-owned tensor comes back as device memory
    assert sorted(p.name for p in (tmp_path / "weights").iterdir()) == sorted(
        e["storage_ref"] + ".nve" for e in doc["layers"])
    torch.save({"keys": keys.cpu(), "bag_keys": bag_keys.cpu(), "offsets": offsets.cpu(), "want": want.cpu(),
                "keys2": keys2.cpu(), "bag_keys2": bag_keys2.cpu(), "offsets2": offsets2.cpu(),
                "want2": want2.cpu()}, tmp_path / "io.pt")
    child = f"""
import sys
sys.path.insert(0, {str(ROOT)!r})
import torch
from nv_embedding_cache_b200 import export as E
io = torch.load({str(tmp_path / 'io.pt')!r})
module, layers = E.load({str(tmp_path)!r})
got = module(io["keys"].cuda(), io["bag_keys"].cuda(), io["offsets"].cuda())
assert torch.equal(got.cpu(), io["want"]), (got.cpu() - io["want"]).abs().max()
got2 = module(io["keys2"].cuda(), io["bag_keys2"].cuda(), io["offsets2"].cuda())
assert torch.equal(got2.cpu(), io["want2"])
assert [type(l).__name__ for l in layers] == ["NVEmbedding", "NVEmbeddingBag"]
print("ok")
"""
    res = subprocess.run([sys.executable, "-c", child], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ))
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_layers_that_share_a_block_are_saved_once_and_come_back_sharing(torch_cuda, tmp_path):
    torch, L = _ops()
    from nv_embedding_cache_b200 import export as E, pynve
    rows, dim = 1200, 8
    block = pynve.ManagedMemBlock(dim, rows, pynve.DataType_t.Float32, [0])
    w = _table(torch, rows, dim, torch.float32)

    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = L.NVEmbedding(rows, dim, torch.float32, L.LayerType.LinearUVM, gpu_cache_size=1 << 20,
                                   storage=block, weight_init=w, id=1)
            self.b = L.NVEmbeddingBag(rows, dim, torch.float32, L.LayerType.LinearUVM, "sum",
                                      gpu_cache_size=1 << 20, storage=block, id=2)

    model = Two()
    E.save_nve(model, str(tmp_path))
    doc = json.loads((tmp_path / "metadata.json").read_text())
    assert len(doc["resources"]["memblocks"]) == 1 and len(list((tmp_path / "weights").iterdir())) == 1
    assert doc["layers"][0]["storage_ref"] == doc["layers"][1]["storage_ref"]
    registry = {}
    a, b = E.load_nve_layers(str(tmp_path), registry=registry)
    assert a.storage is b.storage and len(registry) == 1
    keys = torch.arange(0, rows, 7, device="cuda")
    assert torch.equal(a(keys), w[keys])
    assert torch.equal(b(keys, torch.arange(0, keys.numel() + 1, device="cuda")), w[keys])
    # a second load with the same registry reuses the block and does not read the file again
    (tmp_path / "weights" / (doc["layers"][0]["storage_ref"] + ".nve")).unlink()
    c, d = E.load_nve_layers(str(tmp_path), registry=registry)
    assert c.storage is a.storage
    assert torch.equal(c(keys), w[keys])
    # hand-edited geometry is caught
    doc["resources"]["memblocks"][doc["layers"][0]["storage_ref"]]["num_rows"] = rows + 1
    (tmp_path / "metadata.json").write_text(json.dumps(doc))
    with pytest.raises(ValueError, match="stale or hand-edited"):
        E.load_nve_layers(str(tmp_path))


@pytest.mark.gpu
def test_one_export_loaded_twice_remapped_and_from_the_legacy_layout(torch_cuda, tmp_path):
    """Two loads of one directory in one process give independent layers under their own markers;
    `resource_remap` lets a second directory reuse a block of the first under another key; the layer
    configuration survives the round trip; the flat metadata of schema 1 loads too."""
    torch, L = _ops()
    from nv_embedding_cache_b200 import export as E
    rows, dim = 900, 16
    w = _table(torch, rows, dim, torch.float16)

    class One(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = L.NVEmbedding(rows, dim, torch.float16, L.LayerType.LinearUVM, gpu_cache_size=1 << 20,
                                     weight_init=w, optimize_for_training=False, id=5,
                                     config={"kernel_mode": 2, "kernel_mode_value_1": 512, "default_row_index": 3})

        def forward(self, keys):
            return self.emb(keys)

    model = One().eval()
    keys = torch.randint(0, rows, (128,), device="cuda")
    want = model(keys)
    E.export(model, (keys,), str(tmp_path / "a"),
             dynamic_shapes={"keys": {0: torch.export.Dim("n", min=2, max=4096)}})
    m1, l1 = E.load(str(tmp_path / "a"))
    m2, l2 = E.load(str(tmp_path / "a"))
    assert l1[0].marker_tensor.data_ptr() != l2[0].marker_tensor.data_ptr()
    assert torch.equal(m1(keys), want) and torch.equal(m2(keys), want)
    cfg = l1[0].config
    assert (cfg.kernel_mode, cfg.kernel_mode_value_1, cfg.default_row_index) == (2, 512, 3)
    # keys past the table come back as the default row, through the loaded graph as well
    beyond = torch.full((4,), rows + 7, dtype=torch.int64, device="cuda")
    assert torch.equal(m1(beyond), w[3].expand(4, dim))
    # an update through one loaded copy does not reach the other: they own separate blocks
    first = keys[:2].contiguous()
    l1[0].update(first, torch.zeros(2, dim, dtype=torch.float16, device="cuda"))
    torch.cuda.synchronize()
    assert torch.equal(m2(first), want[:2]) and not torch.equal(m1(first), want[:2])

    # second directory, same block under another key: the registry entry of the first serves it
    E.save_nve(model, str(tmp_path / "b"))
    doc_a = json.loads((tmp_path / "a" / "metadata.json").read_text())
    doc_b = json.loads((tmp_path / "b" / "metadata.json").read_text())
    key_a, key_b = doc_a["layers"][0]["storage_ref"], doc_b["layers"][0]["storage_ref"]
    registry = {}
    (la,) = E.load_nve_layers(str(tmp_path / "a"), registry=registry)
    (lb,) = E.load_nve_layers(str(tmp_path / "b"), registry=registry, resource_remap={key_b: key_a})
    assert la.storage is lb.storage and list(registry) == [key_a]

    # schema 1: a flat list, the table under the module path
    legacy = [dict(doc_a["layers"][0])]
    legacy[0].pop("storage_ref")
    old = tmp_path / "v1"
    (old / "weights").mkdir(parents=True)
    (old / "metadata.json").write_text(json.dumps(legacy))
    (old / "weights" / "emb.nve").write_bytes((tmp_path / "a" / "weights" / (key_a + ".nve")).read_bytes())
    (lv1,) = E.load_nve_layers(str(old))
    assert torch.equal(lv1(keys), want)



@pytest.mark.gpu
def test_ops_from_several_threads_and_streams(torch_cuda):
    """Lookups through the registry run concurrently: four threads, each on a stream of its own,
    against two layers, while a fifth thread registers and unregisters other layers."""
    import threading
    torch, L = _ops()
    rows, dim = 5000, 32
    w = [_table(torch, rows + i, dim, torch.float32)[:rows].contiguous() for i in range(2)]
    layers = [L.NVEmbedding(rows, dim, torch.float32, L.LayerType.GPULayer, weight_init=w[i],
                            optimize_for_training=False) for i in range(2)]
    errors, stop = [], threading.Event()

    def reader(tid):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            rng = np.random.default_rng(tid)
            with torch.cuda.stream(stream):
                for it in range(60):
                    which = (tid + it) % 2
                    keys = torch.from_numpy(rng.integers(0, rows, 777)).cuda(non_blocking=False)
                    got = torch.ops.nve_ops.embedding_lookup(layers[which].marker_tensor, keys, dim,
                                                             layers[which].dtype_tag)
                    stream.synchronize()
                    if not torch.equal(got, w[which][keys]):
                        errors.append(f"thread {tid} iteration {it}: wrong rows")
                        return
        except Exception as e:                      # noqa: BLE001 - reported by the main thread
            errors.append(f"thread {tid}: {e!r}")

    def churn():
        try:
            torch.cuda.set_device(0)
            while not stop.is_set():
                tmp = L.NVEmbedding(64, 8, torch.float32, L.LayerType.GPULayer, optimize_for_training=False)
                del tmp
        except Exception as e:                      # noqa: BLE001
            errors.append(f"churn: {e!r}")

    threads = [threading.Thread(target=reader, args=(i,)) for i in range(4)]
    side = threading.Thread(target=churn)
    side.start()
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    stop.set()
    side.join(60)
    assert not errors, errors
