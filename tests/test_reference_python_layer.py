"""The reference's own Python layer (python/pynve/torch/nve_layers.py, unmodified, imported from
the reference checkout where that exists) over this library's binding module: ``pynve.nve`` is bound
to ``nv_embedding_cache_b200.pynve`` before the reference package is imported, so its plain-Python
path (HAS_TORCH_OPS false) calls straight into libnve_b200.

Without a GPU: the module imports, and every name it takes from the binding exists.  With a GPU and
the checkout on the same machine: its NVEmbedding / NVEmbeddingBag train beside torch.nn.Embedding /
torch.nn.EmbeddingBag, as the reference's tests/python_binding/test_pytorch.py:533-552 does.
"""
import ast
import importlib
import sys

import numpy as np
import pytest

from oracle import build as oracle_build

REF_PY = oracle_build.REFERENCE / "python"
LAYERS_SRC = REF_PY / "pynve" / "torch" / "nve_layers.py"


def _need_checkout():
    if not LAYERS_SRC.exists():
        pytest.skip("the reference checkout is not on this machine")


@pytest.fixture()
def reference_layers():
    """pynve.torch.nve_layers of the reference with pynve.nve bound to this library's module."""
    _need_checkout()
    import nv_embedding_cache_b200.pynve as binding
    saved = {k: v for k, v in sys.modules.items() if k == "pynve" or k.startswith("pynve.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, str(REF_PY))
    try:
        import pynve                                     # the reference's pure-Python package
        sys.modules["pynve.nve"] = binding
        pynve.nve = binding
        yield importlib.import_module("pynve.torch.nve_layers")
    finally:
        sys.path.remove(str(REF_PY))
        for k in [k for k in sys.modules if k == "pynve" or k.startswith("pynve.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_every_binding_name_the_reference_layer_uses_exists():
    _need_checkout()
    import nv_embedding_cache_b200.pynve as binding
    wanted = set()
    for name in ("nve_layers.py", "nve_ops.py", "nve_tensors.py"):
        tree = ast.parse((LAYERS_SRC.parent / name).read_text())
        for node in ast.walk(tree):
            if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id == "nve":
                wanted.add(node.attr)
    assert {"GPUEmbedding", "LinearUVMEmbedding", "UserMemBlock", "ManagedMemBlock", "EmbedLayerConfig",
            "DataType_t", "PoolingType_t"} <= wanted
    missing = sorted(n for n in wanted if not hasattr(binding, n))
    assert not missing, f"the reference layer uses pynve.nve.{missing} which this binding lacks"
    # methods the layer and its autograd functions call on a layer object (`self.emb_layer.f(...)`
    # in the module, `nve_op = weight.emb_layer; nve_op.f(...)` in the autograd functions)
    calls = set()
    for name in ("nve_layers.py", "nve_ops.py", "nve_tensors.py"):
        tree = ast.parse((LAYERS_SRC.parent / name).read_text())
        for node in ast.walk(tree):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute)):
                continue
            target = node.func.value
            if (isinstance(target, ast.Attribute) and target.attr == "emb_layer") or \
                    (isinstance(target, ast.Name) and target.id in ("nve_op", "cache")):
                calls.add(node.func.attr)
    assert {"lookup", "lookup_with_pooling", "concat_backprop", "pooling_backprop", "insert"} <= calls
    lacking = sorted(m for m in calls if not hasattr(binding.NVEmbedBinding, m))
    assert not lacking, f"layer methods missing from the binding: {lacking}"


def test_reference_module_imports_over_this_binding(reference_layers):
    import nv_embedding_cache_b200.pynve as binding
    assert reference_layers.nve is binding
    assert reference_layers.HAS_TORCH_OPS is False
    for name in ("NVEmbedding", "NVEmbeddingBag", "LayerType"):
        assert hasattr(reference_layers, name)
    import torch
    assert reference_layers.torch_type_to_nve_type(torch.float16) == binding.DataType_t.Float16


@pytest.mark.gpu
@pytest.mark.parametrize("layer_type", ["GPULayer", "LinearUVM"])
def test_reference_layers_train_beside_torch(reference_layers, torch_cuda, layer_type):
    torch = torch_cuda
    L = reference_layers
    rows, dim, steps = 2000, 32, 4
    g = torch.Generator(device="cuda").manual_seed(5)
    w0 = (torch.randint(-8, 9, (rows, dim), generator=g, device="cuda") / 16.0).float()
    kind = getattr(L.LayerType, layer_type)
    kw = dict(gpu_cache_size=1 << 20) if layer_type == "LinearUVM" else {}
    emb = L.NVEmbedding(rows, dim, torch.float32, kind, weight_init=w0.clone(), device=torch.device("cuda"), **kw)
    bag = L.NVEmbeddingBag(rows, dim, torch.float32, kind, mode="sum", weight_init=w0.clone(),
                           device=torch.device("cuda"), **kw)
    t_emb = torch.nn.Embedding(rows, dim, sparse=True, device="cuda")
    t_bag = torch.nn.EmbeddingBag(rows, dim, mode="sum", sparse=True, include_last_offset=True, device="cuda")
    with torch.no_grad():
        t_emb.weight.copy_(w0)
        t_bag.weight.copy_(w0)
    opts = [torch.optim.SGD(m.parameters(), lr=0.5) for m in (emb, bag, t_emb, t_bag)]
    rng = np.random.default_rng(3)
    for _ in range(steps):
        keys = torch.from_numpy(rng.integers(0, rows, 64 * 4)).cuda()
        offs = torch.arange(0, 64 * 4 + 1, 4, device="cuda")
        outs = [emb(keys), bag(keys, offs), t_emb(keys), t_bag(keys, offs)]
        assert torch.equal(outs[0], outs[2])
        assert torch.equal(outs[1], outs[3])
        for o, opt in zip(outs, opts):
            opt.zero_grad()
            (o * 0.25).sum().backward()
            opt.step()
    torch.cuda.synchronize()
    probe = torch.arange(rows, device="cuda")
    assert torch.equal(emb(probe), t_emb(probe))
