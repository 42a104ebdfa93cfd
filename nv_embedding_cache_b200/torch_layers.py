"""torch.nn modules over the lookup path, with the names and arguments of the reference's
``pynve.torch.nve_layers`` (python/pynve/torch/nve_layers.py:110-556): ``LayerType``,
``NVEmbedding`` (torch.nn.Embedding-like) and ``NVEmbeddingBag`` (torch.nn.EmbeddingBag-like, CSR
offsets with the trailing sentinel), trainable with any torch optimizer that handles sparse
gradients.  Forward and backward run through the pynve-named edge (``pynve.py``) and so through the
C ABI of the library; the autograd functions are those of the reference's plain-Python path
(``CacheEmbeddingOp`` / ``CacheEmbeddingBagOp``, python/pynve/torch/nve_ops.py:229-316).

Where the compiled op library is present (``HAS_TORCH_OPS``), forward goes through the torch custom
ops ``nve_ops::embedding_lookup`` / ``nve_ops::embedding_lookup_with_pooling`` instead, which
``torch.export`` can trace: every layer owns a one-element marker tensor whose address names it in
the library's registry, and the ops find the layer by that address (reference nve_layers.py:310-327,
nve_ops.py:66-221).  ``nv_embedding_cache_b200.export`` saves and reloads such models.

Provided layer types: ``GPULayer`` (dense table in HBM) and ``LinearUVM`` (GPU cache in front of a
host-resident table).  ``Hierarchical`` and ``HostLayer`` need host tables and parameter servers,
which are outside this library: they raise NotImplementedError.
"""
from __future__ import annotations

import builtins
from enum import Enum
from typing import Optional

import torch

from . import pynve as nve


HAS_TORCH_OPS = nve.load_torch_ops()

# value types a layer can hold, both ways (the binding's enum <-> torch)
_TORCH_OF_NVE = {nve.DataType_t.Float32: torch.float32, nve.DataType_t.Float16: torch.float16}
_NVE_OF_TORCH = {t: n for n, t in _TORCH_OF_NVE.items()}


def nve_type_to_torch_type(nve_type):
    try:
        return _TORCH_OF_NVE[nve.DataType_t(nve_type)]
    except (KeyError, ValueError):
        raise ValueError(f"no torch dtype for layer value type {nve_type!r}") from None


def torch_type_to_nve_type(torch_type: torch.dtype):
    try:
        return _NVE_OF_TORCH[torch_type]
    except KeyError:
        raise ValueError(f"layers hold float32 or float16 rows, not {torch_type}") from None


def pooling_type_from_mode(mode: str, weighted: bool):
    """'sum' / 'mean' (weighted forms with per-sample weights); 'concat' is handled by the caller
    and 'max' does not exist (reference nve_ops.py:32-48)."""
    if mode == "sum":
        return nve.PoolingType_t.WeightedSum if weighted else nve.PoolingType_t.Sum
    if mode == "mean":
        return nve.PoolingType_t.WeightedMean if weighted else nve.PoolingType_t.Mean
    raise ValueError(f"Unsupported pooling mode {mode!r}; expected 'sum' or 'mean' "
                     "('concat' is handled separately). 'max' pooling is not implemented.")


def _flat_tensor(name: str, t: torch.Tensor, dtypes) -> None:
    """The binding reads `t` through its address: it has to be of a type the kernels know and
    dense in memory."""
    if t.dtype not in dtypes:
        wanted = " or ".join(str(d).replace("torch.", "") for d in dtypes)
        raise TypeError(f"{name}: expected a {wanted} tensor, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous tensor (a strided view would be misread)")


def _check_forward_inputs(keys, offsets=None, per_sample_weights=None):
    """Argument checks of a forward call, before any address is handed to the library (the same
    conditions the reference checks, nve_layers.py:42-71)."""
    _flat_tensor("keys", keys, (torch.int64,))
    if offsets is not None:
        _flat_tensor("offsets", offsets, (torch.int64,))
        if offsets.numel() < 2:
            raise ValueError("offsets: at least two entries are needed, bag starts followed by the total "
                             "number of keys (the include_last_offset=True layout)")
    if per_sample_weights is not None:
        _flat_tensor("per_sample_weights", per_sample_weights, (torch.float32, torch.float16))
        if per_sample_weights.numel() != keys.numel():
            raise ValueError(f"per_sample_weights: {per_sample_weights.numel()} weights for "
                             f"{keys.numel()} keys (one weight per key is needed)")


def _stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def config_to_nve_config(config: Optional[dict]):
    cfg = nve.EmbedLayerConfig()
    if config is None:
        return cfg
    for name in ("kernel_mode", "logging_interval", "kernel_mode_value_1", "kernel_mode_value_2",
                 "max_modify_size", "default_row_index", "insert_heuristic"):
        if name in config:
            setattr(cfg, name, config[name])
    if len(config.get("default_embedding", ())) > 0:      # a reloaded config carries the empty default
        raise ValueError("config['default_embedding'] is only supported for HostLayer and Hierarchical layers")
    return cfg


class LayerType(Enum):
    GPULayer = 1
    LinearUVM = 2
    Hierarchical = 3
    HostLayer = 4


class CachedTable(torch.nn.parameter.Parameter):
    """The weight of a layer: a Parameter that carries the layer object, so that an optimizer's
    in-place sparse update goes to the cache and the table through the layer
    (reference nve_tensors.py:19-76)."""

    def __new__(cls, *args, **kwargs):
        if "cache" not in kwargs:
            raise Exception("building a CachedTable Tensor require a viable cache argument")
        cache = kwargs.pop("cache")
        instance = super().__new__(cls, *args, **kwargs)
        instance.emb_layer = cache
        return instance

    def __getstate__(self):
        state = dict(self.__dict__)
        state["emb_layer"] = None        # a native handle: not part of a pickled state
        return state

    def add_(self, other: torch.Tensor, *, alpha: float = 1):
        """What SGD calls with the sparse gradient: rows ``other * alpha`` are accumulated into
        the table (and the cached copies) by the layer."""
        factored = (other * alpha).coalesce() if other.is_sparse else None
        if factored is None:
            raise TypeError("CachedTable.add_ takes a sparse gradient")
        values = factored._values().contiguous()
        keys = factored._indices().reshape(-1).contiguous()
        self.emb_layer.accumulate(keys.numel(), keys.data_ptr(), values.data_ptr(),
                                  _stream_handle(values.device))
        return self


class CacheEmbeddingOp(torch.autograd.Function):
    """Un-pooled lookup; backward = unique keys + per-key gradient sums as a sparse gradient."""

    @staticmethod
    def forward(keys: torch.Tensor, weight: CachedTable):
        result = torch.empty(keys.numel(), weight.shape[-1], dtype=weight.dtype, device=keys.device)
        weight.emb_layer.lookup(keys.numel(), keys.data_ptr(), result.data_ptr(), _stream_handle(keys.device))
        return result

    @staticmethod
    def setup_context(ctx, inputs, output):
        keys, weight = inputs
        ctx.save_for_backward(keys, weight)

    @staticmethod
    def backward(ctx, grad_output):
        keys, weight = ctx.saved_tensors
        num_keys = keys.numel()
        grad_output = grad_output.contiguous()
        unique_keys = torch.empty(num_keys, dtype=torch.int64, device=keys.device)
        result = torch.empty(num_keys, grad_output.shape[-1], dtype=grad_output.dtype, device=keys.device)
        num_unique = weight.emb_layer.concat_backprop(num_keys, keys.data_ptr(), grad_output.data_ptr(),
                                                      unique_keys.data_ptr(), result.data_ptr(),
                                                      _stream_handle(keys.device))
        # unique keys come out sorted and distinct: the gradient is coalesced as built
        return None, torch.sparse_coo_tensor(unique_keys[:num_unique].reshape(1, -1), result[:num_unique],
                                             weight.shape, device=weight.device, check_invariants=False,
                                             is_coalesced=True)


def _weight_type(per_sample_weights):
    if per_sample_weights is None or per_sample_weights.dtype == torch.float32:
        return nve.DataType_t.Float32
    return nve.DataType_t.Float16


class CacheEmbeddingBagOp(torch.autograd.Function):
    """Pooled lookup over CSR bags; backward = pooled backward as a sparse gradient."""

    @staticmethod
    def forward(keys, weight: CachedTable, offsets, mode: str, per_sample_weights):
        result = torch.empty(offsets.numel() - 1, weight.shape[-1], dtype=weight.dtype, device=keys.device)
        pool = pooling_type_from_mode(mode, weighted=per_sample_weights is not None)
        weight.emb_layer.lookup_with_pooling(
            keys.numel(), keys.data_ptr(), result.data_ptr(), int(pool), offsets.numel(), offsets.data_ptr(),
            int(_weight_type(per_sample_weights)),
            per_sample_weights.data_ptr() if per_sample_weights is not None else 0, _stream_handle(keys.device))
        return result

    @staticmethod
    def setup_context(ctx, inputs, output):
        keys, weight, offsets, mode, per_sample_weights = inputs
        ctx.mode = mode
        ctx.save_for_backward(keys, weight, offsets, per_sample_weights)

    @staticmethod
    def backward(ctx, grad_output):
        keys, weight, offsets, per_sample_weights = ctx.saved_tensors
        num_keys = keys.numel()
        grad_output = grad_output.contiguous()
        unique_keys = torch.empty(num_keys, dtype=torch.int64, device=keys.device)
        result = torch.empty(num_keys, grad_output.shape[-1], dtype=grad_output.dtype, device=keys.device)
        pool = pooling_type_from_mode(ctx.mode, weighted=per_sample_weights is not None)
        num_unique = weight.emb_layer.pooling_backprop(
            num_keys, keys.data_ptr(), grad_output.data_ptr(), unique_keys.data_ptr(), result.data_ptr(),
            int(pool), offsets.numel() - 1, offsets.data_ptr(), int(_weight_type(per_sample_weights)),
            per_sample_weights.data_ptr() if per_sample_weights is not None else 0, _stream_handle(keys.device))
        grad = torch.sparse_coo_tensor(unique_keys[:num_unique].reshape(1, -1), result[:num_unique],
                                       weight.shape, device=weight.device, check_invariants=False,
                                       is_coalesced=True)
        return None, grad, None, None, None


def _register_shape_functions() -> None:
    """Shape inference of the two ops for tracing (fake tensors carry no data, so the registry is
    not consulted: rows and type come from the arguments baked into the call).  Another module in
    the process may have registered the same functions already; that registration is kept."""
    def lookup_shape(marker, keys, embedding_size, dtype):
        return keys.new_empty((keys.numel(), embedding_size), dtype=nve_type_to_torch_type(dtype))

    def pooled_shape(marker, keys, offsets, weights, pooling_type, embedding_size, dtype):
        torch._check(offsets.size(0) >= 2, lambda: "offsets: at least two entries are needed")
        return keys.new_empty((offsets.size(0) - 1, embedding_size), dtype=nve_type_to_torch_type(dtype))

    for name, fn in (("nve_ops::embedding_lookup", lookup_shape),
                     ("nve_ops::embedding_lookup_with_pooling", pooled_shape)):
        try:
            torch.library.register_fake(name)(fn)
        except RuntimeError:
            pass


if HAS_TORCH_OPS:
    _register_shape_functions()


def _sparse_rows(unique_keys, rows, count, weight):
    return torch.sparse_coo_tensor(unique_keys[:count].reshape(1, -1), rows[:count], weight.shape,
                                   device=weight.device, check_invariants=False, is_coalesced=True)


class MarkerLookupOp(torch.autograd.Function):
    """Un-pooled lookup through ``nve_ops::embedding_lookup``.  ``weight`` is the layer's CachedTable
    when gradients are wanted (it takes no part in the forward computation, it receives the sparse
    gradient) and None for inference, where backward is refused."""

    @staticmethod
    def forward(marker, keys, weight, embedding_size: int, dtype_tag: int):
        return torch.ops.nve_ops.embedding_lookup(marker, keys, embedding_size, dtype_tag)

    @staticmethod
    def setup_context(ctx, inputs, output):
        _, keys, weight, _, _ = inputs
        ctx.trainable = weight is not None
        if ctx.trainable:
            ctx.save_for_backward(keys, weight)

    @staticmethod
    def backward(ctx, grad_output):
        if not ctx.trainable:
            raise RuntimeError("this layer was built with optimize_for_training=False: it has no backward")
        keys, weight = ctx.saved_tensors
        num_keys = keys.numel()
        grad_output = grad_output.contiguous()
        unique_keys = torch.empty(num_keys, dtype=torch.int64, device=keys.device)
        rows = torch.empty(num_keys, grad_output.shape[-1], dtype=grad_output.dtype, device=keys.device)
        count = weight.emb_layer.concat_backprop(num_keys, keys.data_ptr(), grad_output.data_ptr(),
                                                 unique_keys.data_ptr(), rows.data_ptr(),
                                                 _stream_handle(keys.device))
        return None, None, _sparse_rows(unique_keys, rows, count, weight), None, None


class MarkerPooledLookupOp(torch.autograd.Function):
    """Pooled lookup through ``nve_ops::embedding_lookup_with_pooling``; ``weight`` as in
    MarkerLookupOp."""

    @staticmethod
    def forward(marker, keys, weight, offsets, per_sample_weights, pooling_type: int, embedding_size: int,
                dtype_tag: int):
        return torch.ops.nve_ops.embedding_lookup_with_pooling(marker, keys, offsets, per_sample_weights,
                                                               pooling_type, embedding_size, dtype_tag)

    @staticmethod
    def setup_context(ctx, inputs, output):
        _, keys, weight, offsets, per_sample_weights, pooling_type, _, _ = inputs
        ctx.trainable = weight is not None
        ctx.pooling_type = pooling_type
        ctx.weighted = per_sample_weights is not None
        if ctx.trainable:
            ctx.save_for_backward(keys, weight, offsets, *([per_sample_weights] if ctx.weighted else []))

    @staticmethod
    def backward(ctx, grad_output):
        if not ctx.trainable:
            raise RuntimeError("this layer was built with optimize_for_training=False: it has no backward")
        keys, weight, offsets, *rest = ctx.saved_tensors
        per_sample_weights = rest[0] if ctx.weighted else None
        num_keys = keys.numel()
        grad_output = grad_output.contiguous()
        unique_keys = torch.empty(num_keys, dtype=torch.int64, device=keys.device)
        rows = torch.empty(num_keys, grad_output.shape[-1], dtype=grad_output.dtype, device=keys.device)
        count = weight.emb_layer.pooling_backprop(
            num_keys, keys.data_ptr(), grad_output.data_ptr(), unique_keys.data_ptr(), rows.data_ptr(),
            ctx.pooling_type, offsets.numel() - 1, offsets.data_ptr(), int(_weight_type(per_sample_weights)),
            per_sample_weights.data_ptr() if per_sample_weights is not None else 0, _stream_handle(keys.device))
        return None, None, _sparse_rows(unique_keys, rows, count, weight), None, None, None, None, None


class NVEmbeddingBase(torch.nn.Module):
    """Common part of NVEmbedding / NVEmbeddingBag (reference NVEmbeddingBase, nve_layers.py:124-401):
    builds the storage, the layer object and the ``weight`` Parameter that ties them together.

    Arguments as in the reference.  ``storage``: a ``pynve.MemBlock`` (``UserMemBlock`` around memory
    the caller owns, ``ManagedMemBlock``) or None, in which case a CUDA tensor (GPULayer) or a
    managed block (LinearUVM) is allocated.  ``weight`` must not be used after the module is gone."""

    def __init__(self, num_embeddings: int, embedding_size: int, data_type: torch.dtype, layer_type: LayerType, *,
                 gpu_cache_size: int = 0, host_cache_size: int = 0, storage=None,
                 weight_init: Optional[torch.Tensor] = None, optimize_for_training: bool = True,
                 device: Optional[torch.device] = None, id: Optional[int] = None, config: Optional[dict] = None):
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device("cuda")
        if dev.type != "cuda":
            raise ValueError(f"NV Embedding layers of this library run on cuda devices, got {dev.type}")
        index = dev.index if dev.index is not None else torch.cuda.current_device()
        # what the caller asked for, under the attribute names users of the reference module read
        self.layer_type, self.config = layer_type, config_to_nve_config(config)
        self.num_embeddings, self.embedding_size = num_embeddings, embedding_size
        self.data_type, self.layer_data_type = data_type, torch_type_to_nve_type(data_type)
        self.gpu_cache_size, self.host_cache_size = gpu_cache_size, host_cache_size
        self.optimize_for_training = optimize_for_training
        self.device_index, self.device = index, torch.device("cuda", index)
        self.id = builtins.id(self) if id is None else id
        if storage is not None and not isinstance(storage, nve.MemBlock):
            raise ValueError(f"{layer_type.name} requires storage to be a MemBlock or None")

        if layer_type == LayerType.GPULayer:
            if storage is None:
                if weight_init is not None:
                    tensor_storage = weight_init.detach().clone().to(device=self.device, dtype=data_type).contiguous()
                else:
                    tensor_storage = torch.empty(num_embeddings, embedding_size, dtype=data_type, device=self.device)
                storage = nve.UserMemBlock(tensor_storage.data_ptr(), tensor_storage.nbytes)
            else:
                tensor_storage = nve.device_tensor(storage.get_ptr(), (num_embeddings, embedding_size), data_type,
                                                   self.device)
                if weight_init is not None:
                    tensor_storage.copy_(weight_init)
            self._keep = tensor_storage
            self.emb_layer = nve.GPUEmbedding(embedding_size, num_embeddings, self.layer_data_type, storage,
                                              self.device_index, self.config)
            self.table_ids = {0: "gpu"}
        elif layer_type == LayerType.LinearUVM:
            if gpu_cache_size == 0:
                raise ValueError("GPU cache size > 0 is required for UVM embedding")
            if storage is None:
                storage = nve.ManagedMemBlock(embedding_size, num_embeddings, self.layer_data_type, [self.device_index])
            # the table lives in host-resident memory that the GPU maps: seen from torch as a CUDA tensor
            tensor_storage = nve.device_tensor(storage.get_ptr(), (num_embeddings, embedding_size), data_type,
                                               self.device)
            if weight_init is not None:
                tensor_storage.copy_(weight_init)
                torch.cuda.synchronize(self.device)
            self.emb_layer = nve.LinearUVMEmbedding(embedding_size, num_embeddings, self.layer_data_type, storage,
                                                    gpu_cache_size, optimize_for_training, self.device_index,
                                                    self.config)
            self.table_ids = {0: "gpu_cache"}
        elif layer_type in (LayerType.Hierarchical, LayerType.HostLayer):
            raise NotImplementedError(f"{layer_type.name}: host tables and parameter servers are outside this library")
        else:
            raise ValueError(f"Unknown layer_type: {layer_type}")
        self.storage = storage
        self.memblock_type = storage.get_type()
        self.weight = CachedTable(tensor_storage, cache=self.emb_layer)
        # The layer's name in the registry of the op library: the address of this one-element buffer.
        # Not part of the state dict; an exported graph carries it as a constant into every op call,
        # and a loader points that constant at the marker of the layer it rebuilt.
        self.register_buffer("marker_tensor", torch.tensor([self.id], dtype=torch.int64, device=self.device),
                             persistent=False)
        self.dtype_tag = int(self.layer_data_type)
        self._registered_marker = None
        if HAS_TORCH_OPS:
            self._registered_marker = self.marker_tensor.data_ptr()
            nve.register_for_torch(self._registered_marker, self.emb_layer)

    def _grad_weight(self):
        return self.weight if self.optimize_for_training else None

    def __del__(self):
        # Also runs while the interpreter shuts down, when torch's own module machinery may be half
        # gone: attributes are cleared past Module.__setattr__ and nothing here may raise.
        try:
            marker = self.__dict__.get("_registered_marker")
            if marker is not None:
                self.__dict__["_registered_marker"] = None
                nve.unregister_from_torch(marker)
        except Exception:
            pass
        try:
            layer = self.__dict__.get("emb_layer")
            if layer is not None:
                self.__dict__["emb_layer"] = None
                layer.close()
        except Exception:
            pass

    def to(self, *args, **kwargs):
        """The table and its cache stay where they were built; other parameters and buffers move."""
        device, dtype, non_blocking, _ = torch._C._nn._parse_to(*args, **kwargs)
        for name, param in self.named_parameters():
            if name != "weight":
                param.data = param.data.to(device, dtype if dtype else param.dtype, non_blocking)
        for name, buf in self.named_buffers():
            if name != "marker_tensor":              # its address is the layer's name: it stays put
                buf.data = buf.data.to(device, dtype if dtype else buf.dtype, non_blocking)
        return self

    def update(self, keys: torch.Tensor, updates: torch.Tensor):
        """Overwrite rows (asynchronous on the current stream)."""
        self.emb_layer.update(keys.numel(), keys.data_ptr(), updates.data_ptr(), _stream_handle(self.device))

    def insert(self, keys: torch.Tensor, values: torch.Tensor, table_id: int):
        """Best-effort insert of rows into the cache table ``table_id``."""
        self.emb_layer.insert(keys.numel(), keys.data_ptr(), values.data_ptr(), table_id, _stream_handle(self.device))

    def clear(self):
        self.emb_layer.clear(_stream_handle(self.device))

    def erase(self, keys: torch.Tensor, table_id: int):
        self.emb_layer.erase(keys.numel(), keys.data_ptr(), table_id, _stream_handle(self.device))

    def load_from_stream(self, stream):
        """Loads this layer's table (the tensor named ``self.id``) from a ``.nve`` stream opened for
        binary reading (reference load_tensor_from_stream); cached copies of the old rows are dropped."""
        import numpy as np
        from . import weight_files
        host = np.empty((self.num_embeddings, self.embedding_size),
                        dtype=np.float32 if self.data_type == torch.float32 else np.float16)
        if not weight_files.read_tensor(stream, self.id, host):
            raise KeyError(f"the file holds no tensor named {self.id}")
        with torch.no_grad():
            self.weight.data.copy_(torch.from_numpy(host))
        if self.layer_type == LayerType.LinearUVM:
            self.clear()
        torch.cuda.synchronize(self.device)

    def save_to_stream(self, stream):
        """Appends this layer's table to a ``.nve`` stream (after ``weight_files.write_header``)."""
        from . import weight_files
        torch.cuda.synchronize(self.device)
        weight_files.write_tensor(stream, self.id, self.weight.detach().cpu().numpy())


class NVEmbedding(NVEmbeddingBase):
    """torch.nn.Embedding-like layer (reference NVEmbedding, nve_layers.py:403-461)."""

    def forward(self, keys: torch.Tensor):
        _check_forward_inputs(keys)
        if HAS_TORCH_OPS:
            return MarkerLookupOp.apply(self.marker_tensor, keys, self._grad_weight(), self.embedding_size,
                                        self.dtype_tag)
        return CacheEmbeddingOp.apply(keys, self.weight)


class NVEmbeddingBag(NVEmbeddingBase):
    """torch.nn.EmbeddingBag-like layer with mode 'sum', 'mean' or 'concat' (reference NVEmbeddingBag,
    nve_layers.py:463-556).  Offsets follow ``include_last_offset=True``: num_bags + 1 entries that
    start at 0 and end with ``len(input)``."""

    def __init__(self, num_embeddings: int, embedding_size: int, data_type: torch.dtype, layer_type: LayerType,
                 mode: str, **kwargs):
        if mode != "concat":
            pooling_type_from_mode(mode, weighted=False)      # fail fast on unsupported modes
        super().__init__(num_embeddings, embedding_size, data_type, layer_type, **kwargs)
        self.mode = mode

    def forward(self, input: torch.Tensor, offsets: torch.Tensor,
                per_sample_weights: Optional[torch.Tensor] = None):
        _check_forward_inputs(input, offsets, per_sample_weights)
        if not HAS_TORCH_OPS:
            if self.mode == "concat":
                return CacheEmbeddingOp.apply(input, self.weight)
            return CacheEmbeddingBagOp.apply(input, self.weight, offsets, self.mode, per_sample_weights)
        if self.mode == "concat":
            return MarkerLookupOp.apply(self.marker_tensor, input, self._grad_weight(), self.embedding_size,
                                        self.dtype_tag)
        pool = pooling_type_from_mode(self.mode, weighted=per_sample_weights is not None)
        return MarkerPooledLookupOp.apply(self.marker_tensor, input, self._grad_weight(), offsets,
                                          per_sample_weights, int(pool), self.embedding_size, self.dtype_tag)
