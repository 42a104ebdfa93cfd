"""torch.nn edge (torch_layers.NVEmbedding / NVEmbeddingBag) against torch.nn.Embedding /
torch.nn.EmbeddingBag, in the manner of the reference's tests/python_binding/test_pytorch.py:
forward outputs over several SGD steps with sparse gradients must agree, for the dense (GPULayer)
and the cached (LinearUVM) layer types, fp32 and fp16."""
import numpy as np
import pytest

from nv_embedding_cache_b200 import datagen as dg


def test_argument_checks_need_no_gpu():
    import torch
    from nv_embedding_cache_b200 import torch_layers as L
    from nv_embedding_cache_b200 import pynve
    assert L.pooling_type_from_mode("sum", False) == pynve.PoolingType_t.Sum
    assert L.pooling_type_from_mode("mean", True) == pynve.PoolingType_t.WeightedMean
    with pytest.raises(ValueError):
        L.pooling_type_from_mode("max", False)
    with pytest.raises(TypeError):
        L._check_forward_inputs(torch.zeros(4, dtype=torch.int32))
    with pytest.raises(ValueError):
        L._check_forward_inputs(torch.zeros(4, dtype=torch.int64), torch.zeros(1, dtype=torch.int64))
    with pytest.raises(ValueError):
        L._check_forward_inputs(torch.zeros(4, dtype=torch.int64), torch.zeros(2, dtype=torch.int64),
                                torch.zeros(3, dtype=torch.float32))
    with pytest.raises(ValueError):
        L.config_to_nve_config({"default_embedding": [0, 0]})
    assert L.config_to_nve_config({"default_embedding": []}).default_embedding == []
    assert L.config_to_nve_config({"kernel_mode": 2, "default_row_index": 5}).default_row_index == 5
    assert L.torch_type_to_nve_type(torch.float16) == pynve.DataType_t.Float16


def train_loop(torch, layer, key_sets, offsets, target, weights=None, lr=0.1):
    """The reference test's loop: forward, MSE loss, backward, SGD step; returns the outputs."""
    loss = torch.nn.MSELoss()
    opt = torch.optim.SGD(layer.parameters(), lr=lr)
    outs = []
    for keys in key_sets:
        if offsets is None:
            out = layer(keys)
        elif weights is None:
            out = layer(keys, offsets)
        else:
            out = layer(keys, offsets, per_sample_weights=weights)
        loss(out, target).backward()
        opt.step()
        opt.zero_grad()
        outs.append(out.detach().clone())
    torch.cuda.synchronize()
    return outs


def make_layers(torch, L, cls, ref_weight, dtype, **kw):
    n, d = ref_weight.shape
    uvm = cls(n, d, dtype, L.LayerType.LinearUVM, gpu_cache_size=4 << 20, weight_init=ref_weight, **kw)
    gpu = cls(n, d, dtype, L.LayerType.GPULayer, weight_init=ref_weight, **kw)
    return uvm, gpu


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name", ["float32", "float16"])
def test_embedding_training_matches_torch(torch_cuda, dtype_name):
    torch = torch_cuda
    from nv_embedding_cache_b200 import torch_layers as L
    dtype = getattr(torch, dtype_name)
    n, d = 10000, 16
    torch.manual_seed(3)
    ref = torch.nn.Embedding(n, d, dtype=dtype, sparse=True, device="cuda")
    uvm, gpu = make_layers(torch, L, L.NVEmbedding, ref.weight, dtype)
    keys = torch.tensor([5, 4, 3, 100, 1024, 6, 5, 5, 100], dtype=torch.int64, device="cuda")   # with repeats
    target = torch.randn(keys.numel(), d, dtype=dtype, device="cuda")
    want = train_loop(torch, ref, [keys] * 6, None, target)
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)
    for layer in (uvm, gpu):
        got = train_loop(torch, layer, [keys] * 6, None, target)
        for a, b in zip(got, want):
            assert torch.allclose(a.float(), b.float(), **tol)
        assert not torch.equal(got[0], got[-1])              # the updates reached the table
    del uvm, gpu


@pytest.mark.gpu
@pytest.mark.parametrize("mode,weighted", [("sum", False), ("mean", False), ("sum", True)])
def test_embedding_bag_training_matches_torch(torch_cuda, mode, weighted):
    torch = torch_cuda
    from nv_embedding_cache_b200 import torch_layers as L
    n, d, bags = 5000, 32, 300
    torch.manual_seed(4)
    ref = torch.nn.EmbeddingBag(n, d, sparse=True, mode=mode, include_last_offset=True, device="cuda")
    uvm, gpu = make_layers(torch, L, L.NVEmbeddingBag, ref.weight, torch.float32, mode=mode)
    _, offsets_np = dg.csr_bags(bags, 0, 12, 5)
    total = int(offsets_np[-1])
    key_sets = [torch.from_numpy(dg.zipf_keys(total, n, 1.1, 40 + s, dg.permutation(n))).cuda() for s in range(5)]
    offsets = torch.from_numpy(offsets_np).cuda()
    weights = torch.rand(total, device="cuda") if weighted else None
    target = torch.randn(bags, d, device="cuda")
    want = train_loop(torch, ref, key_sets, offsets, target, weights)
    for layer in (uvm, gpu):
        got = train_loop(torch, layer, key_sets, offsets, target, weights)
        for a, b in zip(got, want):
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)
    # the tables themselves ended up equal to torch's weight
    assert torch.allclose(gpu.weight.detach(), ref.weight.detach(), rtol=1e-4, atol=1e-5)
    assert torch.allclose(uvm.weight.detach(), ref.weight.detach(), rtol=1e-4, atol=1e-5)
    del uvm, gpu


@pytest.mark.gpu
def test_bag_fp16_concat_and_modify_calls(torch_cuda):
    torch = torch_cuda
    from nv_embedding_cache_b200 import pynve, torch_layers as L
    n, d = 2000, 8
    w = torch.randn(n, d, device="cuda").half()
    # fp16 pooled forward + backward (pooled gradients summed in fp32, rounded once)
    bag = L.NVEmbeddingBag(n, d, torch.float16, L.LayerType.GPULayer, "sum", weight_init=w)
    keys = torch.tensor([1, 2, 3, 3, 7, 1], dtype=torch.int64, device="cuda")
    offsets = torch.tensor([0, 2, 4, 6], dtype=torch.int64, device="cuda")
    out = bag(keys, offsets)
    want = torch.stack([w[1].float() + w[2].float(), w[3].float() * 2, w[7].float() + w[1].float()]).half()
    assert torch.allclose(out.float(), want.float(), rtol=2e-3, atol=2e-3)
    out.sum().backward()
    g = bag.weight.grad.coalesce()
    assert sorted(g.indices().reshape(-1).tolist()) == [1, 2, 3, 7]
    dense = dict(zip(g.indices().reshape(-1).tolist(), g.values().float().sum(dim=1).tolist()))
    assert dense == {1: 2.0 * d, 2: 1.0 * d, 3: 2.0 * d, 7: 1.0 * d}
    # concat mode is the plain lookup
    cat = L.NVEmbeddingBag(n, d, torch.float16, L.LayerType.GPULayer, "concat", weight_init=w)
    assert torch.equal(cat(keys, offsets), w[keys])
    # update / erase / clear / insert on a cached layer over caller-owned storage
    table = torch.zeros(n, d, dtype=torch.float32).pin_memory()
    layer = L.NVEmbedding(n, d, torch.float32, L.LayerType.LinearUVM, gpu_cache_size=1 << 20,
                          storage=pynve.UserMemBlock(table.data_ptr(), table.nbytes), optimize_for_training=False)
    k = torch.tensor([1, 2, 3, 4, 5], dtype=torch.int64, device="cuda")
    upd = torch.arange(1.0, 1.0 + 5 * d, device="cuda").reshape(5, d)
    layer.update(k, upd)
    torch.cuda.synchronize()
    assert torch.equal(layer(k), upd)
    assert torch.equal(table[1:6], upd.cpu())                 # written through to the caller's memory
    layer.insert(k, upd, 0)
    layer.erase(k[:2], 0)
    layer.clear()
    torch.cuda.synchronize()
    assert torch.equal(layer(k), upd)
    with pytest.raises(NotImplementedError):
        L.NVEmbedding(n, d, torch.float32, L.LayerType.HostLayer, optimize_for_training=False)
    with pytest.raises(ValueError):
        L.NVEmbedding(n, d, torch.float32, L.LayerType.LinearUVM)
    del bag, cat, layer


@pytest.mark.gpu
def test_layers_save_and_load_weight_files(torch_cuda, tmp_path):
    """Two layers written to one .nve file and read back into fresh layers by id, as the reference's
    multi-layer load test does; the cached layer must not serve rows it cached before the load."""
    torch = torch_cuda
    from nv_embedding_cache_b200 import torch_layers as L, weight_files
    n, d = 3000, 8
    a = L.NVEmbedding(n, d, torch.float32, L.LayerType.GPULayer, weight_init=torch.randn(n, d), id=1)
    b = L.NVEmbedding(n, d, torch.float16, L.LayerType.LinearUVM, gpu_cache_size=1 << 20,
                      weight_init=torch.randn(n, d).half(), id=2, optimize_for_training=False)
    path = tmp_path / "model.nve"
    with open(path, "wb+") as f:
        weight_files.write_header(f)
        a.save_to_stream(f)
        b.save_to_stream(f)
    a2 = L.NVEmbedding(n, d, torch.float32, L.LayerType.GPULayer, id=1)
    b2 = L.NVEmbedding(n, d, torch.float16, L.LayerType.LinearUVM, gpu_cache_size=1 << 20, id=2,
                       weight_init=torch.zeros(n, d).half(), optimize_for_training=False)
    keys = torch.arange(0, n, 7, dtype=torch.int64, device="cuda")
    b2.insert(keys, b2(keys), 0)                  # stale rows (zeros) in the cache before the load
    with open(path, "rb") as f:
        b2.load_from_stream(f)
        a2.load_from_stream(f)
    assert torch.equal(a2(keys), a(keys)) and torch.equal(b2(keys), b(keys))
    assert torch.equal(a2.weight.detach(), a.weight.detach())
    with open(path, "rb") as f, pytest.raises(KeyError):
        L.NVEmbedding(n, d, torch.float32, L.LayerType.GPULayer, id=3).load_from_stream(f)
    del a, b, a2, b2
