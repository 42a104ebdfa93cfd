"""The reference's own Python layer (python/pynve/torch/{nve_layers,nve_ops,nve_export}.py,
unmodified, imported from the reference checkout where that exists) over this library's binding
module: ``pynve.nve`` is bound to ``nv_embedding_cache_b200.pynve`` before the reference package is
imported.

Each case runs in a child interpreter, because importing the reference package registers shape
functions for the torch ops process-wide.  Two settings: with the compiled op library
(HAS_TORCH_OPS true: the reference's marker / custom-op / export path) and with
NVE_B200_TORCH_OPS=0 (its plain-Python path).

Without a GPU: the modules import, and every name they take from the binding exists.  With a GPU and
the checkout on the same machine: NVEmbedding / NVEmbeddingBag train beside torch.nn.Embedding /
torch.nn.EmbeddingBag, as the reference's tests/python_binding/test_pytorch.py:533-552 does, and a
model goes through the reference's export / load.
"""
import ast
import os
import subprocess
import sys
from pathlib import Path

import pytest

from oracle import build as oracle_build

ROOT = Path(__file__).resolve().parent.parent
REF_PY = oracle_build.REFERENCE / "python"
TORCH_DIR = REF_PY / "pynve" / "torch"
PY_FILES = ("nve_layers.py", "nve_ops.py", "nve_tensors.py", "nve_export.py")

PRELUDE = f"""
import sys
sys.path.insert(0, {str(ROOT)!r})
sys.path.insert(0, {str(REF_PY)!r})
import nv_embedding_cache_b200.pynve as binding
import pynve                      # the reference's pure-Python package
sys.modules["pynve.nve"] = binding
pynve.nve = binding
import pynve.torch as pt
import pynve.torch.nve_layers as L
"""


def _need_checkout():
    if not TORCH_DIR.exists():
        pytest.skip("the reference checkout is not on this machine")


def _run(body: str, torch_ops: bool, timeout: int = 600) -> str:
    env = dict(os.environ, NVE_B200_TORCH_OPS="1" if torch_ops else "0")
    res = subprocess.run([sys.executable, "-c", PRELUDE + body], env=env, capture_output=True, text=True,
                         timeout=timeout)
    assert res.returncode == 0, res.stdout + "\n" + res.stderr
    return res.stdout


def _names_taken_from_binding(files, aliases):
    wanted = set()
    for name in files:
        tree = ast.parse((TORCH_DIR / name).read_text())
        for node in ast.walk(tree):
            if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id in aliases:
                wanted.add(node.attr)
    return wanted


def test_every_binding_name_the_reference_layer_uses_exists():
    _need_checkout()
    import nv_embedding_cache_b200.pynve as binding
    wanted = _names_taken_from_binding(PY_FILES, {"nve", "_nve_mod"})
    assert {"GPUEmbedding", "LinearUVMEmbedding", "UserMemBlock", "ManagedMemBlock", "EmbedLayerConfig",
            "DataType_t", "PoolingType_t", "TensorFileFormat", "write_tensor_to_stream", "MemBlockType",
            "resolve_memblock_devices", "HostMemBlock", "LinearMemBlock", "register_for_torch"} <= wanted
    missing = sorted(n for n in wanted if not hasattr(binding, n))
    assert not missing, f"the reference layer uses pynve.nve.{missing} which this binding lacks"
    # methods the layer and its autograd functions call on a layer object (`self.emb_layer.f(...)`
    # in the module, `nve_op = weight.emb_layer; nve_op.f(...)` in the autograd functions)
    calls = set()
    for name in PY_FILES:
        tree = ast.parse((TORCH_DIR / name).read_text())
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
    # what the export module reads from a block type and a config object
    assert {m.name for m in binding.MemBlockType} == {"Linear", "NVL", "MPI", "Managed", "User", "Host"}
    assert callable(binding.EmbedLayerConfig().to_json)


def test_reference_modules_import_on_the_plain_path():
    _need_checkout()
    out = _run("""
assert L.nve is binding
assert pt.HAS_TORCH_OPS is False
for name in ("NVEmbedding", "NVEmbeddingBag", "LayerType"):
    assert hasattr(L, name)
import torch
assert L.torch_type_to_nve_type(torch.float16) == binding.DataType_t.Float16
print("ok")
""", torch_ops=False)
    assert "ok" in out


def test_reference_modules_import_over_the_op_library():
    """Importing the binding loads the compiled ops, so the reference package sees them, registers its
    shape functions for them and offers its export module."""
    _need_checkout()
    out = _run("""
import torch
assert pt.HAS_TORCH_OPS is True
import pynve.torch.nve_export as E
schema = str(torch.ops.nve_ops.embedding_lookup_with_pooling.default._schema)
assert schema == ("nve_ops::embedding_lookup_with_pooling(Tensor marker, Tensor keys, Tensor offsets, "
                  "Tensor? weights, int pooling_type, int embedding_size, int dtype) -> Tensor"), schema
# the reference's shape functions answer for fake tensors through this library's op definitions
from torch._subclasses.fake_tensor import FakeTensorMode
with FakeTensorMode():
    marker = torch.zeros(1, dtype=torch.int64)
    keys = torch.zeros(12, dtype=torch.int64)
    offsets = torch.zeros(5, dtype=torch.int64)
    a = torch.ops.nve_ops.embedding_lookup(marker, keys, 16, int(binding.DataType_t.Float16))
    b = torch.ops.nve_ops.embedding_lookup_with_pooling(marker, keys, offsets, None, 1, 16,
                                                        int(binding.DataType_t.Float32))
    assert a.shape == (12, 16) and a.dtype == torch.float16
    assert b.shape == (4, 16) and b.dtype == torch.float32
for name in ("save_nve", "export", "export_aot", "load_nve_layers", "load", "load_aot"):
    assert callable(getattr(E, name))
print("ok")
""", torch_ops=True)
    assert "ok" in out


TRAIN = """
import numpy as np, torch
layer_type = {layer_type!r}
rows, dim, steps = 2000, 32, 4
g = torch.Generator(device="cuda").manual_seed(5)
w0 = (torch.randint(-8, 9, (rows, dim), generator=g, device="cuda") / 16.0).float()
kind = getattr(L.LayerType, layer_type)
kw = dict(gpu_cache_size=1 << 20) if layer_type == "LinearUVM" else {{}}
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
print("ok")
"""


@pytest.mark.gpu
@pytest.mark.parametrize("torch_ops", [False, True])
@pytest.mark.parametrize("layer_type", ["GPULayer", "LinearUVM"])
def test_reference_layers_train_beside_torch(torch_cuda, layer_type, torch_ops):
    _need_checkout()
    assert "ok" in _run(TRAIN.format(layer_type=layer_type), torch_ops=torch_ops)


@pytest.mark.gpu
def test_reference_export_and_load_over_this_binding(torch_cuda, tmp_path):
    _need_checkout()
    out = _run(f"""
import torch
import pynve.torch.nve_export as E

class Model(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = L.NVEmbedding(500, 16, torch.float32, L.LayerType.GPULayer, optimize_for_training=False,
                                 weight_init=torch.arange(500 * 16, dtype=torch.float32).reshape(500, 16) / 8, id=11)
        self.head = torch.nn.Linear(16, 4)
    def forward(self, keys):
        return self.head(self.emb(keys))

model = Model().cuda().eval()
keys = torch.randint(0, 500, (64,), device="cuda")
want = model(keys)
E.export(model, (keys,), {str(tmp_path)!r})
module, layers = E.load({str(tmp_path)!r})
assert torch.equal(module(keys), want)
print("ok")
""", torch_ops=True)
    assert "ok" in out
