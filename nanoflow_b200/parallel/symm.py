"""Symmetric heap: one device allocation per rank, mapped into every peer process with CUDA IPC, so
that a buffer has the same byte offset on all GPUs and kernels can load / store peer memory directly
over NVLink. ``torch.distributed`` is used once, to exchange the 64-byte IPC handles.

This is the B200-side counterpart of the reference's MSCCL++ registered memory + SmChannel setup
(pipeline/include/netWrapper.cuh:31-139, pipeline/src/pipeline.cu:293-337), with one process per GPU
instead of one thread per GPU.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch

from .. import ops as _ops


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}
        self._owner = owner


class SymmetricHeap:
    def __init__(self, rank: int, world: int, device: torch.device, nbytes: int, group=None):
        import torch.distributed as dist

        self.rank, self.world, self.device = rank, world, device
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        lib = _ops.lib()
        torch.cuda.set_device(device)
        base = ctypes.c_void_p()
        rc = lib.nfk_symm_alloc(ctypes.byref(base), ctypes.c_longlong(self.nbytes))
        if rc != 0:
            raise RuntimeError(f"symmetric heap allocation of {self.nbytes >> 20} MiB failed")
        self.base = base.value
        handle = (ctypes.c_ubyte * 64)()
        if lib.nfk_ipc_get_handle(ctypes.c_void_p(self.base), handle) != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        handles: List[bytes] = [None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        self.peer_base: List[int] = []
        for r in range(world):
            if r == rank:
                self.peer_base.append(self.base)
                continue
            out = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
            if lib.nfk_ipc_open_handle(buf, ctypes.byref(out)) != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed (peer access unavailable?)")
            self.peer_base.append(out.value)
        self._bump = 0
        self._bytes_view = torch.as_tensor(_CudaArray(self.base, self.nbytes, self), device=device)
        if world > 1:
            dist.barrier(group=group)

    def alloc_bytes(self, nbytes: int, align: int = 256) -> int:
        off = (self._bump + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise RuntimeError(f"symmetric heap exhausted ({self.nbytes >> 20} MiB)")
        self._bump = off + nbytes
        return off

    def alloc(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = self.alloc_bytes(max(nbytes, 16))
        t = self._bytes_view[off:off + nbytes].view(dtype).view(*shape)
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor is not inside the symmetric heap")
        return off

    def close(self) -> None:
        lib = _ops.lib()
        for r, p in enumerate(self.peer_base):
            if r != self.rank and p:
                lib.nfk_ipc_close_handle(ctypes.c_void_p(p))
        self.peer_base = []
