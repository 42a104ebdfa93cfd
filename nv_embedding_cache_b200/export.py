"""Saving and reloading models that contain NVEmbedding / NVEmbeddingBag layers.

On disk, the layout and the ``metadata.json`` schema (version 2) of the reference's
``pynve.torch.nve_export`` (python/pynve/torch/nve_export.py:201-360,418-760), so that a directory
written by either side loads on the other::

    save_dir/
      metadata.json        {"version": 2, "resources": {"remote_ps": {}, "memblocks": {...}}, "layers": [...]}
      weights/<key>.nve    one .nve container per storage block, tensor named by the layer id
      model.pt2            torch.export program (export) or AOTInductor package (export_aot)

A layer's table is written once per storage block: layers that share a block share the file, and
come back sharing one block.  A block around memory the caller owned (``UserMemBlock``) cannot be
named in a file; it is rebuilt as the kind of block every layer that used it can work with
(device memory for GPULayer alone or with LinearUVM, managed memory for LinearUVM alone).

The exported graph holds each layer's marker tensor as a constant.  ``load`` rebuilds the layers
(which registers their own markers with the op library), materialises the graph once and points
each marker constant at the live layer's marker, so every op call finds its layer.
"""
from __future__ import annotations

import builtins
import json
import os
from typing import Optional

import torch

from . import pynve as nve
from .torch_layers import (HAS_TORCH_OPS, LayerType, NVEmbedding, NVEmbeddingBag, NVEmbeddingBase,
                           torch_type_to_nve_type)

METADATA_SCHEMA_VERSION = 2
_SERIALISABLE = (nve.MemBlockType.User, nve.MemBlockType.Host, nve.MemBlockType.Linear, nve.MemBlockType.Managed)


def _need_ops(what: str) -> None:
    if not HAS_TORCH_OPS:
        raise RuntimeError(f"{what} needs the compiled op library (libnve_b200_torch_ops.so): build it with "
                           "`python -m nv_embedding_cache_b200.build`")


def _dtype_name(dtype: torch.dtype) -> str:
    return str(dtype).removeprefix("torch.")


def _dtype_of(name: str) -> torch.dtype:
    return getattr(torch, name.removeprefix("torch."))


def _nve_layers(model: torch.nn.Module):
    return [(path, m) for path, m in model.named_modules() if isinstance(m, NVEmbeddingBase)]


def _block_kind_for(users: set) -> str:
    """Kind of block that replaces a caller-owned one, from the layer types that used it."""
    if users <= {LayerType.GPULayer, LayerType.LinearUVM} and LayerType.GPULayer in users:
        return nve.MemBlockType.Linear.name
    if users == {LayerType.LinearUVM}:
        return nve.MemBlockType.Managed.name
    raise ValueError(f"no block kind serves layer types {sorted(t.name for t in users)} together")


def _describe(model: torch.nn.Module):
    """(document for metadata.json, {id(storage) -> resource key})."""
    blocks: dict[str, dict] = {}
    key_of: dict[int, str] = {}
    users_of_user_block: dict[str, set] = {}
    layers = []
    for path, m in _nve_layers(model):
        storage = m.storage
        if not isinstance(storage, nve.MemBlock):
            raise ValueError(f"layer '{path}': only block-backed layers (GPULayer, LinearUVM) can be saved")
        kind = m.memblock_type
        if kind not in _SERIALISABLE:
            raise ValueError(f"layer '{path}': a block of type {kind} does not describe its placement and "
                             "cannot be saved")
        key = key_of.setdefault(builtins.id(storage), f"mb-{builtins.id(storage)}")
        blocks.setdefault(key, {"type": kind.name, "row_elements": m.embedding_size, "num_rows": m.num_embeddings,
                                "dtype": _dtype_name(m.data_type)})
        if kind == nve.MemBlockType.User:
            users_of_user_block.setdefault(key, set()).add(m.layer_type)
        layers.append({
            "id": m.id, "module_path": path, "num_embeddings": m.num_embeddings,
            "embedding_size": m.embedding_size, "dtype": _dtype_name(m.data_type),
            "layer_type": m.layer_type.name, "gpu_cache_size": m.gpu_cache_size,
            "host_cache_size": m.host_cache_size, "optimize_for_training": m.optimize_for_training,
            "is_bag": isinstance(m, NVEmbeddingBag), "mode": getattr(m, "mode", None),
            "storage_ref": key, "config": json.loads(m.config.to_json()),
        })
    for key, users in users_of_user_block.items():
        blocks[key]["type"] = _block_kind_for(users)
    doc = {"version": METADATA_SCHEMA_VERSION, "resources": {"remote_ps": {}, "memblocks": blocks},
           "layers": layers}
    return doc, key_of


def save_nve(model: torch.nn.Module, save_dir: str) -> None:
    """Writes metadata.json and weights/*.nve for every NVEmbedding layer of `model`."""
    os.makedirs(os.path.join(save_dir, "weights"), exist_ok=True)
    doc, key_of = _describe(model)
    with open(os.path.join(save_dir, "metadata.json"), "w") as f:
        json.dump(doc, f, indent=2)
    written = set()
    for _, m in _nve_layers(model):
        key = key_of[builtins.id(m.storage)]
        if key in written:
            continue
        written.add(key)
        with open(os.path.join(save_dir, "weights", key + ".nve"), "wb") as f:
            nve.TensorFileFormat().write_table_file_header(f)
            nve.write_tensor_to_stream(m.emb_layer, f, m.id)


def export(model: torch.nn.Module, example_inputs, save_dir: str, *, dynamic_shapes=None) -> None:
    """save_nve + the torch.export program of `model` as model.pt2."""
    _need_ops("export")
    save_nve(model, save_dir)
    program = torch.export.export(model, example_inputs, dynamic_shapes=dynamic_shapes)
    torch.export.save(program, os.path.join(save_dir, "model.pt2"))


def export_aot(model: torch.nn.Module, example_inputs, save_dir: str, *, dynamic_shapes=None,
               inductor_configs: Optional[dict] = None) -> None:
    """save_nve + an AOTInductor package of `model` as model.pt2.  Runtime constant folding is
    switched on so that the marker buffers stay constants a loader can re-point (they would
    otherwise be baked into the generated code)."""
    _need_ops("export_aot")
    save_nve(model, save_dir)
    configs = {"aot_inductor.use_runtime_constant_folding": True} | (inductor_configs or {})
    program = torch.export.export(model, example_inputs, dynamic_shapes=dynamic_shapes)
    torch._inductor.aoti_compile_and_package(program, package_path=os.path.join(save_dir, "model.pt2"),
                                             inductor_configs=configs)


def _build_block(desc: dict, device_index: int):
    kind, rows, cols = desc["type"], desc["num_rows"], desc["row_elements"]
    dtype = torch_type_to_nve_type(_dtype_of(desc["dtype"]))
    if kind == "Host":
        return nve.HostMemBlock(cols, rows, dtype)
    if kind == "Linear":
        return nve.LinearMemBlock(cols, rows, dtype, nve.resolve_memblock_devices(nve.MemBlockType.Linear,
                                                                                   device_index)[0])
    if kind == "Managed":
        return nve.ManagedMemBlock(cols, rows, dtype, nve.resolve_memblock_devices(nve.MemBlockType.Managed,
                                                                                    device_index))
    raise ValueError(f"cannot rebuild a block of type {kind!r}; Host, Linear and Managed blocks can be")


def load_nve_layers(save_dir: str, *, gpu_cache_size_override: Optional[int] = None,
                    device: Optional[torch.device] = None, registry: Optional[dict] = None,
                    resource_remap: Optional[dict] = None) -> list:
    """Rebuilds the layers a directory describes, tables loaded.  `registry` (resource key ->
    block), when passed to several calls, lets models saved from one process share blocks again;
    `resource_remap` renames keys of the file before they are looked up in it.  The flat metadata
    of schema 1 (a list of layers, each with storage of its own) is read as well.  The caller keeps
    the returned layers alive for as long as a graph refers to them."""
    _need_ops("load_nve_layers")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.type != "cuda":
        raise ValueError("layers of this library live on a cuda device")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    with open(os.path.join(save_dir, "metadata.json")) as f:
        doc = json.load(f)
    if isinstance(doc, list):
        # the flat layout of schema 1: one entry per layer, no resources section, every layer with
        # storage of its own and its table in weights/<module path with dots as underscores>.nve
        doc = {"version": 1, "layers": doc}
    if doc.get("version", 1) > METADATA_SCHEMA_VERSION:
        raise RuntimeError(f"metadata.json has schema version {doc['version']}; this reader knows up to "
                           f"{METADATA_SCHEMA_VERSION}")
    registry = {} if registry is None else registry
    remap = resource_remap or {}
    described = doc.get("resources", {}).get("memblocks", {})

    layers = []
    for entry in doc["layers"]:
        path, rows, cols = entry["module_path"], entry["num_embeddings"], entry["embedding_size"]
        kind = LayerType[entry["layer_type"]]
        if kind not in (LayerType.GPULayer, LayerType.LinearUVM):
            raise NotImplementedError(f"layer '{path}': {kind.name} layers are outside this library")
        ref = entry.get("storage_ref")
        if doc.get("version", 1) < 2:
            # schema 1: the layer allocates its own storage; the file is named after the module path
            ref, key, fresh, storage = path.replace(".", "_"), None, True, None
        else:
            if not ref:
                raise ValueError(f"layer '{path}' names no storage block")
            key = remap.get(ref, ref)
            desc = described.get(key)
            if desc is not None and (desc["row_elements"], desc["num_rows"]) != (cols, rows):
                raise ValueError(f"block '{key}' is {desc['num_rows']} x {desc['row_elements']} but layer '{path}' "
                                 f"expects {rows} x {cols}: stale or hand-edited metadata?")
            fresh = key not in registry
            if fresh:
                if desc is None:
                    raise ValueError(f"storage_ref '{key}' is not among resources.memblocks")
                registry[key] = _build_block(desc, device.index)
            storage = registry[key]
        kwargs = dict(optimize_for_training=entry["optimize_for_training"], device=device, id=entry["id"],
                      config=entry.get("config"), storage=storage)
        if kind == LayerType.LinearUVM:
            kwargs["gpu_cache_size"] = (entry["gpu_cache_size"] if gpu_cache_size_override is None
                                        else gpu_cache_size_override)
        data_type = _dtype_of(entry["dtype"])
        if entry.get("is_bag", False):
            layer = NVEmbeddingBag(rows, cols, data_type, kind, entry.get("mode"), **kwargs)
        else:
            layer = NVEmbedding(rows, cols, data_type, kind, **kwargs)
        if fresh:       # a block found in the registry already holds its rows
            with open(os.path.join(save_dir, "weights", ref + ".nve"), "rb") as f:
                layer.load_from_stream(f)
        layer._export_module_path = path
        layers.append(layer)
    return layers


def load(save_dir: str, *, gpu_cache_size_override: Optional[int] = None, device: Optional[torch.device] = None):
    """(module, layers) of a directory written by export: the graph of model.pt2 as a callable module
    whose marker constants point at the rebuilt layers.  Keep `layers` alive while the module is in
    use."""
    layers = load_nve_layers(save_dir, gpu_cache_size_override=gpu_cache_size_override, device=device)
    module = torch.export.load(os.path.join(save_dir, "model.pt2")).module()
    for layer in layers:
        path = layer._export_module_path
        owner = module.get_submodule(path) if path else module
        owner.marker_tensor = layer.marker_tensor
    return module, layers


def _point_markers(loader, layers) -> None:
    known = set(loader.get_constant_fqns())
    for layer in layers:
        path = layer._export_module_path
        name = f"{path}.marker_tensor" if path else "marker_tensor"
        if name not in known:
            raise RuntimeError(f"the package has no updatable constant '{name}' (it has {sorted(known)}); it was "
                               "probably built without runtime constant folding: use export_aot")
        for inactive_buffer in (False, True):
            loader.load_constants({name: layer.marker_tensor}, inactive_buffer, False, True)


def load_aot(save_dir: str, *, gpu_cache_size_override: Optional[int] = None,
             device: Optional[torch.device] = None):
    """(loader, layers) of a directory written by export_aot; run it with ``loader.run([inputs...])``.
    Both constant buffers of the package are pointed at the live markers, without copying them."""
    _need_ops("load_aot")
    from torch._C._aoti import AOTIModelPackageLoader
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    layers = load_nve_layers(save_dir, gpu_cache_size_override=gpu_cache_size_override,
                             device=torch.device("cuda", index))
    loader = AOTIModelPackageLoader(os.path.join(save_dir, "model.pt2"), "model", False, 1, index)
    _point_markers(loader, layers)
    return loader, layers


def rebind_markers(loader, layers) -> None:
    """Points the marker constants at the layers again, after the package's constant buffers were
    rebuilt or swapped (which replaces the markers by copies)."""
    _point_markers(loader, layers)
