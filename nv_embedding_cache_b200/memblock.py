"""Host-resident table storage that the GPU kernels read in place.

``ManagedMemBlock`` mirrors the reference's class of the same name (``src/memblock.cpp:108-135``,
exposed to Python by its binding): managed memory with the host as preferred location and the
listed GPUs as accessors.  It is the storage to use for the backing table of the cached
(LinearUVM) layer: GPU kernels keep the host link's rate over the whole table, which memory from
``cudaHostAlloc`` / ``tensor.pin_memory()`` does not beyond a few GB.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import capi


def copy_bytes(dst: int, src: int, nbytes: int) -> None:
    """Synchronous byte copy between any two addresses the process can name (host, pinned, managed
    or device memory): the runtime works out the direction.  Without a CUDA driver only host
    addresses exist, and a plain memmove does."""
    if not torch.cuda.is_available():
        C.memmove(dst, src, nbytes)
        return
    runtime = C.CDLL("libcudart.so.12")      # already in the process: torch loaded it
    runtime.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    runtime.cudaMemcpy.restype = C.c_int
    err = runtime.cudaMemcpy(dst, src, nbytes, 4)     # 4 = cudaMemcpyDefault
    if err != 0:
        raise RuntimeError(f"cudaMemcpy of {nbytes} bytes failed with error {err}")


class ManagedMemBlock:
    """``ManagedMemBlock(size_in_bytes, gpu_ids)`` or, as the reference binding also offers,
    ``ManagedMemBlock(row_size, num_embeddings, elem_bytes, gpu_ids)`` through :meth:`for_table`."""

    TYPE = "Managed"

    @classmethod
    def for_table(cls, row_size: int, num_embeddings: int, elem_bytes: int, gpu_ids=(0,)):
        return cls(row_size * num_embeddings * elem_bytes, gpu_ids)

    def __init__(self, size_in_bytes: int, gpu_ids=(0,)):
        ids = (C.c_int32 * len(gpu_ids))(*gpu_ids)
        p = C.c_void_p()
        capi.check(capi.lib.nve_b200_managed_block_create(C.byref(p), size_in_bytes, ids, len(gpu_ids)))
        self.ptr = p.value
        self.size = size_in_bytes

    def get_ptr(self) -> int:
        return self.ptr

    def get_size_in_bytes(self) -> int:
        return self.size

    def get_handle(self) -> int:
        return self.ptr

    def get_type(self) -> str:
        return self.TYPE

    def copy_from(self, src) -> None:
        """Copy a C-contiguous buffer (numpy array, tensor on any device) to the start of the block."""
        t = src if isinstance(src, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(src))
        if not t.is_contiguous():
            raise ValueError("copy_from: source buffer must be C-contiguous")
        nbytes = t.numel() * t.element_size()
        if nbytes > self.size:
            raise IndexError(f"copy_from: source is {nbytes} bytes but memblock holds {self.size} bytes")
        self.as_tensor((t.numel(),), t.dtype).copy_(t.reshape(-1))
        torch.cuda.synchronize()

    def data_ptr(self) -> int:          # so that a block can be passed wherever a tensor is accepted
        return self.ptr

    def as_tensor(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """A CPU tensor over the block (no copy).  The block must outlive the tensor."""
        count = int(np.prod(shape))
        itemsize = torch.empty((), dtype=dtype).element_size()
        if count * itemsize > self.size:
            raise ValueError("shape does not fit the block")
        raw = (C.c_uint8 * (count * itemsize)).from_address(self.ptr)
        return torch.frombuffer(raw, dtype=dtype, count=count).view(*shape)

    def close(self):
        if self.ptr:
            capi.check(capi.lib.nve_b200_managed_block_destroy(self.ptr))
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
