"""Python edge with the class and method names of the reference's pynve bindings
(python/pynve/bindings/python_binding.cu:150-391, binding_layers.hpp:72-440), served by the C ABI
of libnve_b200.  Arguments are raw addresses and raw ``cudaStream_t`` values, exactly as in the
pybind layer, so ``pynve.torch.nve_layers`` style callers pass ``tensor.data_ptr()`` and
``torch.cuda.current_stream().cuda_stream``.
"""
from __future__ import annotations

import ctypes as C
import enum

from . import capi
from .layers import ExecutionContext, GpuTable, GPUEmbeddingLayer, LinearUVMEmbeddingLayer, _Layer


class DataType_t(enum.IntEnum):
    Unknown = capi.DTYPE_UNKNOWN
    Float32 = capi.DTYPE_FLOAT32
    Float16 = capi.DTYPE_FLOAT16


class PoolingType_t(enum.IntEnum):
    Concatenate = capi.POOL_CONCATENATE
    Sum = capi.POOL_SUM
    Mean = capi.POOL_MEAN
    WeightedSum = capi.POOL_WEIGHTED_SUM
    WeightedMean = capi.POOL_WEIGHTED_MEAN


class EmbedLayerConfig:
    """reference binding_layers.hpp:50-65"""

    def __init__(self):
        self.logging_interval = -1
        self.kernel_mode = 0
        self.kernel_mode_value_1 = 0
        self.kernel_mode_value_2 = 0
        self.max_modify_size = 1 << 20
        self.default_row_index = -1
        self.default_embedding = []     # host and hierarchical layers only (not provided here)
        # cached layer only: "default" = the reference's default insert heuristic (automatic cache
        # population, threshold 0.75), "never", or a float threshold
        self.insert_heuristic = "default"

    def to_json(self) -> str:
        """The fields the reference serialises (binding_layers.hpp:62-65), as a JSON object; what a
        loader hands back to ``config_to_nve_config``."""
        import json
        return json.dumps({name: getattr(self, name) for name in (
            "logging_interval", "kernel_mode", "kernel_mode_value_1", "kernel_mode_value_2", "max_modify_size",
            "default_row_index")} | {"default_embedding": [int(b) for b in self.default_embedding]})


_POOL_NAME = {PoolingType_t.Concatenate: "concatenate", PoolingType_t.Sum: "sum",
              PoolingType_t.Mean: "mean", PoolingType_t.WeightedSum: "weighted_sum",
              PoolingType_t.WeightedMean: "weighted_mean"}
MAX_RUN_SIZE = 1024  # reference binding_layers.hpp:390


class NVEmbedBinding:
    """Common lookup / modify / backward surface (reference NVEmbedBinding<int64_t>)."""

    def __init__(self, layer: _Layer, row_size: int, data_type: DataType_t, device_id: int):
        self._layer = layer
        self._dtype = DataType_t(data_type)
        self._row_elems = row_size
        self._row_bytes = row_size * (4 if self._dtype == DataType_t.Float32 else 2)
        self._device = device_id
        self._ctx: dict[int, ExecutionContext] = {}
        self._deduper = None
        self._dedup_capacity = 0
        self._runs = (C.c_int64 * 2)()

    # one execution context per caller stream, created on first use (binding_layers.hpp:352-367)
    def _context(self, stream: int) -> ExecutionContext:
        ctx = self._ctx.get(stream)
        if ctx is None:
            ctx = self._layer.create_execution_context(stream or None, stream or None)
            self._ctx[stream] = ctx
        return ctx

    def get_embedding_dim(self) -> int:
        return self._row_elems

    def get_data_type(self) -> DataType_t:
        return self._dtype

    def lookup(self, num_keys: int, keys: int, output: int, stream: int = 0) -> None:
        self._layer.lookup(self._context(stream), num_keys, keys, output, self._row_bytes)

    def lookup_with_pooling(self, num_keys: int, keys: int, output: int, pooling_type: int,
                            num_offsets: int, offsets: int, weight_data_type: int, weights: int,
                            stream: int = 0) -> None:
        self._layer.lookup_pooled(self._context(stream), num_keys, keys, output, self._row_bytes,
                                  _POOL_NAME[PoolingType_t(pooling_type)], int(self._dtype),
                                  csr_offsets=offsets, num_csr_offsets=num_offsets,
                                  weights=weights or None, weight_type=int(weight_data_type))

    def accumulate(self, num_keys: int, keys: int, updates: int, stream: int = 0) -> None:
        self._layer.accumulate(self._context(stream), num_keys, keys, self._row_bytes,
                               self._row_bytes, updates, int(self._dtype), -1)

    def update(self, num_keys: int, keys: int, updates: int, stream: int = 0) -> None:
        self._layer.update(self._context(stream), num_keys, keys, self._row_bytes, self._row_bytes,
                           updates, -1)

    def insert(self, num_keys: int, keys: int, values: int, table_id: int = 0, stream: int = 0) -> None:
        self._layer.insert(self._context(stream), num_keys, keys, self._row_bytes, self._row_bytes,
                           values, table_id)

    def clear(self, stream: int = 0) -> None:
        self._layer.clear(self._context(stream))

    def erase(self, num_keys: int, keys: int, table_id: int = 0, stream: int = 0) -> None:
        self._layer.erase(self._context(stream), num_keys, keys, table_id)

    def concat_backprop(self, num_keys: int, keys: int, grads: int, unique_keys: int,
                        output_grads: int, stream: int = 0) -> int:
        """Backward of an un-pooled lookup: unique keys and the per-key sum of the incoming
        gradient rows.  Returns the number of unique keys (binding_layers.hpp:131-189).
        Scratch (inverse map, offsets, chunk map) is owned by this object and grows on demand."""
        self._ensure_deduper(num_keys)
        s = stream or None
        capi.check(capi.lib.nve_b200_deduper_dedup(
            self._deduper, keys, num_keys, unique_keys, self._counts.data_ptr(),
            self._loc_map.data_ptr(), self._runs, self._inverse.data_ptr(), self._offsets.data_ptr(),
            s, 0))
        if self._dtype != DataType_t.Float32:        # fp16 rows: added in fp16, as the reference does
            capi.check(capi.lib.nve_b200_dedup_grads_f16(
                self._deduper, grads, self._row_bytes, self._row_bytes, num_keys,
                self._inverse.data_ptr(), self._offsets.data_ptr(), self._loc_map.data_ptr(),
                output_grads, self._row_bytes, s))
            return int(self._runs[0])
        capi.check(capi.lib.nve_b200_dedup_grads(
            self._deduper, grads, self._row_bytes, self._row_bytes, num_keys, unique_keys,
            self._inverse.data_ptr(), self._offsets.data_ptr(), self._loc_map.data_ptr(),
            output_grads, self._row_bytes, 0, 0, 1.0, s))
        return int(self._runs[0])

    def _ensure_deduper(self, num_keys: int):
        import torch
        if num_keys > self._dedup_capacity:
            if self._deduper:
                capi.check(capi.lib.nve_b200_deduper_destroy(self._deduper))
            self._deduper = C.c_void_p()
            capi.check(capi.lib.nve_b200_deduper_create(C.byref(self._deduper), capi.KEY_INT64,
                                                        MAX_RUN_SIZE, num_keys))
            dev = torch.device("cuda", self._device)
            cap = num_keys + num_keys // MAX_RUN_SIZE + 2
            self._counts = torch.empty(num_keys + 1, dtype=torch.int64, device=dev)
            self._inverse = torch.empty(num_keys + 1, dtype=torch.int64, device=dev)
            self._offsets = torch.empty(cap + 1, dtype=torch.int64, device=dev)
            self._loc_map = torch.empty(cap + 1, dtype=torch.int64, device=dev)
            self._dedup_capacity = num_keys

    def pooling_backprop(self, num_keys: int, keys: int, grads: int, unique_keys: int, output_grads: int,
                         pooling_type: int, num_offsets: int, offsets: int, data_type: int = 0,
                         weights: int = 0, stream: int = 0) -> int:
        """Backward of a pooled lookup (binding_layers.hpp:191-250): ``grads`` holds one row per bag
        in the layer's data type, ``offsets`` the int64 CSR offsets of ``num_offsets`` bags
        (``num_offsets + 1`` entries), ``weights`` optional per-key weights (``data_type``: Float32
        or Float16).  Writes the unique keys and, per unique key, the weighted sum of the gradients
        of the bags it occurs in; returns the number of unique keys.

        Float32 layers with Float32 weights run on the caller's buffers.  Float16 gradients or
        weights are widened to fp32, summed in fp32 and rounded to fp16 once at the end (the
        reference multiplies and adds them in fp16: its sums carry one rounding per addition)."""
        self._ensure_deduper(num_keys)
        n_unique = C.c_int64(0)
        half_rows = self._dtype != DataType_t.Float32
        half_weights = bool(weights) and int(data_type) == int(DataType_t.Float16)
        if not half_rows and not half_weights:
            capi.check(capi.lib.nve_b200_pooling_backprop(
                self._deduper, num_keys, keys, grads, self._row_bytes, self._row_bytes, int(pooling_type),
                capi.SPARSE_CSR, offsets, num_offsets, 0, weights or None, unique_keys, output_grads,
                self._row_bytes, C.byref(n_unique), stream or None))
            return int(n_unique.value)
        import torch
        dev = torch.device("cuda", self._device)
        width = self._row_elems
        with torch.cuda.stream(torch.cuda.ExternalStream(stream, device=dev) if stream else
                               torch.cuda.default_stream(dev)):
            g = device_tensor(grads, (num_offsets, width), torch.float16 if half_rows else torch.float32, dev).float()
            w = None
            if weights:
                w = device_tensor(weights, (num_keys,), torch.float16 if half_weights else torch.float32, dev).float()
            out32 = torch.empty((num_keys, width), dtype=torch.float32, device=dev)
            capi.check(capi.lib.nve_b200_pooling_backprop(
                self._deduper, num_keys, keys, g.data_ptr(), width * 4, width * 4, int(pooling_type),
                capi.SPARSE_CSR, offsets, num_offsets, 0, w.data_ptr() if w is not None else None, unique_keys,
                out32.data_ptr(), width * 4, C.byref(n_unique), stream or None))
            u = int(n_unique.value)
            out = device_tensor(output_grads, (num_keys, width), torch.float16 if half_rows else torch.float32, dev)
            out[:u].copy_(out32[:u])
        return u

    def close(self) -> None:
        for ctx in self._ctx.values():
            ctx.wait()
            ctx.destroy()
        self._ctx.clear()
        if self._deduper:
            capi.check(capi.lib.nve_b200_deduper_destroy(self._deduper))
            self._deduper = None
        self._layer.destroy()


class _DevicePointer:
    """Raw device address described through the CUDA array interface, so torch can wrap it."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 3, "strides": None}


def device_tensor(ptr: int, shape, dtype, device):
    """A torch tensor over device-accessible memory at ``ptr`` (no copy; the memory must outlive it)."""
    import torch
    typestr = {torch.float32: "<f4", torch.float16: "<f2", torch.int64: "<i8", torch.uint8: "|u1"}[dtype]
    t = torch.as_tensor(_DevicePointer(ptr, shape, typestr), device=device)
    if t.data_ptr() != int(ptr):
        raise RuntimeError("memory at this address belongs to another device than the one asked for")
    return t


class MemBlockType(str, enum.Enum):
    """What MemBlock.get_type() answers with (reference binding enum, python_binding.cu:229-236).
    Members compare equal to their names, so ``block.get_type() == "Managed"`` also holds."""
    Linear = "Linear"
    NVL = "NVL"
    MPI = "MPI"
    Managed = "Managed"
    User = "User"
    Host = "Host"

    def __str__(self) -> str:
        return self.value


def _element_bytes(data_type) -> int:
    return 4 if DataType_t(data_type) == DataType_t.Float32 else 2


class MemBlock:
    """Storage handed to a layer (reference MemBlock, include/memblock.hpp): an address, a size and
    a type.  The owner of the memory keeps it alive for as long as the layer lives."""

    TYPE = MemBlockType.User

    def __init__(self, ptr: int, size_in_bytes: int):
        self._ptr = int(ptr)
        self._size = int(size_in_bytes)

    def get_ptr(self) -> int:
        return self._ptr

    def get_handle(self) -> int:
        return self._ptr

    def get_size_in_bytes(self) -> int:
        return self._size

    def get_type(self) -> MemBlockType:
        return self.TYPE

    def data_ptr(self) -> int:
        return self._ptr

    def copy_from(self, src) -> None:
        """Byte copy of a C-contiguous buffer (numpy array, bytes, ...) into the block, bounds-checked
        (reference python_binding.cu:243-262).  Host, managed and device memory alike."""
        import numpy as np
        a = np.asarray(src)
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError("copy_from: source buffer must be C-contiguous")
        if a.nbytes > self._size:
            raise IndexError(f"copy_from: source is {a.nbytes} bytes but memblock holds {self._size} bytes")
        if a.nbytes:
            from .memblock import copy_bytes
            copy_bytes(self._ptr, a.ctypes.data, a.nbytes)


class UserMemBlock(MemBlock):
    """Memory the caller owns: ``UserMemBlock(tensor.data_ptr(), tensor.nbytes)``."""

    def __init__(self, ptr: int, size: int):
        super().__init__(ptr, size)


class ManagedMemBlock(MemBlock):
    """Managed memory kept on the host and mapped into the listed GPUs, with the reference binding's
    signature: ``ManagedMemBlock(row_size, num_embeddings, data_type, gpu_ids)``."""

    TYPE = MemBlockType.Managed

    def __init__(self, row_size: int, num_embeddings: int, data_type: DataType_t, gpu_ids=(0,)):
        from .memblock import ManagedMemBlock as _Block
        self._block = _Block(row_size * num_embeddings * _element_bytes(data_type), tuple(gpu_ids))
        super().__init__(self._block.get_ptr(), self._block.get_size_in_bytes())

    def copy_from(self, src) -> None:
        self._block.copy_from(src)

    def as_tensor(self, shape, dtype):
        return self._block.as_tensor(shape, dtype)

    def close(self) -> None:
        self._block.close()


class LinearMemBlock(MemBlock):
    """Plain device memory on one GPU: ``LinearMemBlock(row_size, num_embeddings, dtype, device_id)``
    (reference python_binding.cu:264-267).  ``device_id = -1``, the reference's host-side form, is
    not provided: use HostMemBlock."""

    TYPE = MemBlockType.Linear

    def __init__(self, row_size: int, num_embeddings: int, dtype: DataType_t, device_id: int = -1):
        if device_id < 0:
            raise NotImplementedError("LinearMemBlock on the host: use HostMemBlock")
        import torch
        self._tensor = torch.empty(row_size * num_embeddings * _element_bytes(dtype), dtype=torch.uint8,
                                   device=torch.device("cuda", device_id))
        super().__init__(self._tensor.data_ptr(), self._tensor.nbytes)


class HostMemBlock(MemBlock):
    """Pinned host memory that every GPU can read in place: ``HostMemBlock(row_size,
    num_embeddings, dtype)`` (reference python_binding.cu:292-294)."""

    TYPE = MemBlockType.Host

    def __init__(self, row_size: int, num_embeddings: int, dtype: DataType_t):
        import torch
        self._tensor = torch.empty(row_size * num_embeddings * _element_bytes(dtype), dtype=torch.uint8,
                                   pin_memory=True)
        super().__init__(self._tensor.data_ptr(), self._tensor.nbytes)


class NVLMemBlock(MemBlock):
    """One allocation spread over several GPUs of one process.  Not provided: a table sharded over
    GPUs is the ShardedEmbeddingTable of this library, one process per GPU."""

    TYPE = MemBlockType.NVL

    def __init__(self, *args, **kwargs):
        raise NotImplementedError("NVLMemBlock: use nv_embedding_cache_b200.sharded.ShardedEmbeddingTable")


def resolve_memblock_devices(type, def_index: int, override=()):
    """GPU ids for rebuilding a block at load time (reference src/memblock.cpp:144-164): `override`
    if given; for NVL every GPU from `def_index` up; otherwise `def_index` alone."""
    if len(override):
        return list(override)
    if MemBlockType(type) == MemBlockType.NVL:
        import torch
        count = torch.cuda.device_count()
        if not 0 <= def_index < count:
            raise ValueError(f"resolve_memblock_devices: def_index={def_index} out of range, system has {count} GPUs")
        return list(range(def_index, count))
    return [def_index]


class Table:
    """Host tables and parameter servers are outside this library; the name exists so that callers
    written against the reference binding can still test ``isinstance(storage, Table)``."""

    def __init__(self, *args, **kwargs):
        raise NotImplementedError("host tables and parameter servers are not part of this library")


class PSType_t(enum.IntEnum):
    """Kinds of parameter-server tables of the reference binding (names only: none is provided)."""
    NVHashMap = 0
    Abseil = 1
    ParallelHash = 2
    Redis = 3


NVHashMap, Abseil, ParallelHash, Redis = PSType_t.NVHashMap, PSType_t.Abseil, PSType_t.ParallelHash, PSType_t.Redis


class ParameterServerTable(Table):
    """Parameter servers are outside this library (see Table)."""


class HierarchicalEmbedding:
    def __init__(self, *args, **kwargs):
        raise NotImplementedError("the hierarchical layer (host and remote tiers) is not part of this library")


class HostEmbedding:
    def __init__(self, *args, **kwargs):
        raise NotImplementedError("the host layer is not part of this library")


def get_dl_tensor(layer: "NVEmbedBinding", data_type):
    """DLPack capsule over the table memory of a layer, [num_embeddings, row_size] of `data_type` on
    the layer's device (reference get_dl_tensor: how the torch layer sees a UVM table)."""
    import torch
    from torch.utils import dlpack
    dt = {DataType_t.Float32: torch.float32, DataType_t.Float16: torch.float16}[DataType_t(data_type)]
    t = device_tensor(_address(layer._memblock), (layer._num_rows, layer._row_elems), dt,
                      torch.device("cuda", layer._device))
    return dlpack.to_dlpack(t)


_TORCH_REGISTRY: dict[int, "NVEmbedBinding"] = {}
_TORCH_OPS_LIBRARY = capi.PACKAGE_DIR / "libnve_b200_torch_ops.so"
_torch_ops_loaded = False


def load_torch_ops() -> bool:
    """Loads the compiled op library (nve_ops::embedding_lookup, nve_ops::embedding_lookup_with_pooling)
    into torch, once.  False when it has not been built or NVE_B200_TORCH_OPS=0 asks for the
    plain-Python path; callers then see HAS_TORCH_OPS false, as with a reference build without its
    torch bindings."""
    global _torch_ops_loaded
    if _torch_ops_loaded:
        return True
    import os
    if os.environ.get("NVE_B200_TORCH_OPS", "1") == "0" or not _TORCH_OPS_LIBRARY.exists():
        return False
    import torch
    torch.ops.load_library(str(_TORCH_OPS_LIBRARY))
    _torch_ops_loaded = True
    return True


def register_for_torch(marker_ptr: int, layer: "NVEmbedBinding") -> None:
    """Names `layer` by the address of its marker tensor in the library's registry, where the torch
    custom ops look it up (reference python_binding.cu:372-377).  The layer object is kept alive
    until unregister_from_torch."""
    capi.check(capi.lib.nve_b200_registry_register(int(marker_ptr), layer._layer.handle, layer._row_elems,
                                                   int(layer._dtype), layer._device))
    _TORCH_REGISTRY[int(marker_ptr)] = layer


def unregister_from_torch(marker_ptr: int) -> None:
    if _TORCH_REGISTRY.pop(int(marker_ptr), None) is not None:
        capi.check(capi.lib.nve_b200_registry_unregister(int(marker_ptr)))


class TensorFileFormat:
    """Writer of the ``.nve`` container's file header (reference binding class of the same name,
    python_binding.cu:196-202)."""

    def write_table_file_header(self, stream) -> None:
        from . import weight_files
        weight_files.write_header(stream)


def _table_view(layer: "NVEmbedBinding"):
    import torch
    dt = torch.float32 if layer._dtype == DataType_t.Float32 else torch.float16
    device = torch.device("cuda", layer._device)
    return device_tensor(_address(layer._memblock), (layer._num_rows, layer._row_elems), dt, device), device


def write_tensor_to_stream(layer: "NVEmbedBinding", stream, name: int) -> None:
    """Appends the table of `layer` as tensor `name` to a .nve container whose header is already
    written (reference write_tensor_to_stream, binding_layers.hpp:626-630,693-703)."""
    import torch
    from . import weight_files
    table, device = _table_view(layer)
    torch.cuda.synchronize(device)
    weight_files.write_tensor(stream, name, table.cpu().numpy())


def load_tensor_from_stream(layer: "NVEmbedBinding", stream, name: int) -> None:
    """Fills the table of `layer` with tensor `name` of a .nve container opened for binary reading
    (reference load_tensor_from_stream as the binding exposes it); rows cached from the old table
    are dropped."""
    import numpy as np
    import torch
    from . import weight_files
    host = np.empty((layer._num_rows, layer._row_elems),
                    dtype=np.float32 if layer._dtype == DataType_t.Float32 else np.float16)
    if not weight_files.read_tensor(stream, name, host):
        raise KeyError(f"the file holds no tensor named {name}")
    table, device = _table_view(layer)
    table.copy_(torch.from_numpy(host))
    torch.cuda.synchronize(device)
    if isinstance(layer, LinearUVMEmbedding):
        layer.clear(torch.cuda.current_stream(device).cuda_stream)


def _address(memblock) -> int:
    return memblock if isinstance(memblock, int) else memblock.data_ptr()


class GPUEmbedding(NVEmbedBinding):
    """Dense table in HBM (reference GPUEmbedding, binding_layers.hpp:665-690).  ``memblock`` is the
    table: a torch tensor (kept alive here) or a raw device address."""

    def __init__(self, row_size: int, num_embeddings: int, data_type: DataType_t, memblock,
                 device_id: int = 0, config: EmbedLayerConfig | None = None):
        config = config or EmbedLayerConfig()
        elem = 4 if DataType_t(data_type) == DataType_t.Float32 else 2
        self._memblock = memblock
        self._num_rows = num_embeddings
        layer = GPUEmbeddingLayer(_address(memblock), num_embeddings, row_size * elem, int(data_type),
                                  device_id=device_id, default_row_index=config.default_row_index)
        super().__init__(layer, row_size, data_type, device_id)


class LinearUVMEmbedding(NVEmbedBinding):
    """GPU cache in front of a linear table in host / managed / device memory (reference
    LinearUVMEmbedding, binding_layers.hpp:534-640)."""

    def __init__(self, row_size: int, num_embeddings: int, data_type: DataType_t, memblock,
                 gpu_cache_size: int, optimize_for_training: bool = True, device_id: int = 0,
                 config: EmbedLayerConfig | None = None):
        config = config or EmbedLayerConfig()
        elem = 4 if DataType_t(data_type) == DataType_t.Float32 else 2
        self._memblock = memblock
        self._num_rows = num_embeddings
        self._table = GpuTable(gpu_cache_size, row_size * elem, int(data_type), device_id=device_id,
                               uvm_table=_address(memblock), uvm_num_rows=num_embeddings,
                               max_modify_size=config.max_modify_size,
                               kernel_mode_type=config.kernel_mode,
                               kernel_mode_value=self._kernel_mode_value(config))
        layer = LinearUVMEmbeddingLayer(self._table, default_row_index=config.default_row_index,
                                        insert_heuristic=getattr(config, "insert_heuristic", "default"))
        super().__init__(layer, row_size, data_type, device_id)

    def _kernel_mode_value(self, config: EmbedLayerConfig) -> int:
        """kernel_mode_value of the table from the two config values (binding_layers.hpp:569-580):
        sort-gather takes the tile size, pipeline gather the address of {task_size, aux streams}."""
        if config.kernel_mode == 2:
            return config.kernel_mode_value_1 if config.kernel_mode_value_1 > 0 else 1024
        if config.kernel_mode == 3:
            self._pipeline_params = (C.c_uint64 * 2)(
                config.kernel_mode_value_1 if config.kernel_mode_value_1 > 0 else 1024,
                config.kernel_mode_value_2 if config.kernel_mode_value_2 > 0 else 16)
            return C.addressof(self._pipeline_params)
        return config.kernel_mode_value_1

    def close(self) -> None:
        super().close()
        self._table.destroy()


# As with the reference, importing the binding module is what makes the torch ops exist.
try:
    load_torch_ops()
except ImportError:        # no torch in this interpreter: the ctypes edge works without it
    pass
