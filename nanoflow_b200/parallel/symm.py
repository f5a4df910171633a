"""Symmetric heap: one device allocation per rank, mapped into every peer process, so that a buffer
has the same byte offset on all GPUs and kernels can load / store peer memory directly over NVLink,
and (``nvls`` form) reduce or broadcast inside the NVSwitch through one multicast address.
``torch.distributed`` is used once, to exchange the handles.

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


def default_backend() -> str:
    """``NANOFLOW_SYMM_BACKEND`` = ``ipc`` | ``nvls`` | ``auto`` (default ``auto``: NVLS when it can be set up)."""
    import os

    return os.environ.get("NANOFLOW_SYMM_BACKEND", "auto").lower()


class SymmetricHeap:
    """Two ways to build the heap:

    ``ipc``   one ``cudaMalloc`` per rank, opened in every peer with CUDA IPC. Peers are reached with
              plain loads / stores. A rank that exits leaves nothing bound in the NVSwitch, so failure
              tests use this form.
    ``nvls``  memory from ``torch.distributed._symmetric_memory`` (driver virtual-memory allocations
              exchanged as file descriptors), which also binds all ranks' heaps to one NVLink multicast
              object: ``mc_base`` is then an address at which ``multimem.ld_reduce`` returns the sum
              over all ranks of the word at that offset and ``multimem.st`` writes every rank's copy.
              Peer pointers work as with ``ipc``. Only the allocation and the handle exchange are the
              library's; every kernel that touches the memory is this package's.
    ``auto``  ``nvls`` if every rank could set it up (and the GPUs report multicast support), else ``ipc``.
    """

    def __init__(self, rank: int, world: int, device: torch.device, nbytes: int, group=None,
                 backend: str = ""):
        import torch.distributed as dist

        self.rank, self.world, self.device = rank, world, device
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.mc_base = 0
        self.backend = "ipc"
        self._symm_tensor = None
        self._symm_handle = None
        backend = (backend or default_backend()) if world > 1 else "ipc"
        if backend not in ("ipc", "nvls", "auto"):
            raise ValueError(f"unknown symmetric heap backend {backend!r}")
        torch.cuda.set_device(device)
        if backend in ("nvls", "auto") and self._try_nvls(group, required=(backend == "nvls")):
            return
        lib = _ops.lib()
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

    def _try_nvls(self, group, required: bool) -> bool:
        """Allocate through torch's symmetric memory and keep the multicast address. All ranks agree on
        the outcome (a MIN all-reduce of "it worked here"), so either all use it or none does."""
        import torch.distributed as dist

        ok, err = 1, ""
        t = hdl = None
        try:
            import torch.distributed._symmetric_memory as symm_mem

            grp = group if group is not None else dist.group.WORLD
            t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(t, grp)
            ptrs = [int(x) for x in hdl.buffer_ptrs]
            mc = int(hdl.multicast_ptr or 0)
            if len(ptrs) != self.world or mc == 0 or ptrs[self.rank] != t.data_ptr():
                ok, err = 0, f"no multicast address (multicast_ptr={mc:#x})"
        except Exception as e:  # noqa: BLE001 - any failure of the optional path means "use CUDA IPC"
            ok, err = 0, f"{type(e).__name__}: {e}"
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) != 1:
            if required:
                raise RuntimeError(f"NVLS symmetric heap unavailable on rank {self.rank}: {err or 'failed on another rank'}")
            del hdl, t
            return False
        t.zero_()
        torch.cuda.synchronize(self.device)
        self._symm_tensor, self._symm_handle = t, hdl
        self.base = t.data_ptr()
        self.peer_base = [int(x) for x in hdl.buffer_ptrs]
        self.mc_base = int(hdl.multicast_ptr)
        self.backend = "nvls"
        self._bump = 0
        self._bytes_view = t
        dist.barrier(group=group)
        return True

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
        if self.backend == "nvls":
            # the mappings go away with the tensor; drop the views first
            self.peer_base, self.mc_base = [], 0
            self._bytes_view = self._symm_handle = self._symm_tensor = None
            return
        lib = _ops.lib()
        for r, p in enumerate(self.peer_base):
            if r != self.rank and p:
                lib.nfk_ipc_close_handle(ctypes.c_void_p(p))
        self.peer_base = []
