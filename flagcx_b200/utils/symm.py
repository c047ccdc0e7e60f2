"""Symmetric (peer-mapped) device buffers exposed as torch tensors.

``SymmetricBuffer`` allocates with flagcxMemAlloc (CUDA VMM, exportable), registers
the allocation as a window with a communicator -- a collective call, every rank
must create its buffers in the same order with the same sizes -- and hands out
torch tensors that alias the memory.  Collectives whose arguments lie inside such a
buffer run without staging copies.
"""
from __future__ import annotations

import torch

from flagcx_b200 import capi


class _CudaArray:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_ptr(ptr: int, nbytes: int, device: int) -> torch.Tensor:
    """uint8 tensor aliasing [ptr, ptr+nbytes) on `device`; the caller keeps the memory alive."""
    return torch.as_tensor(_CudaArray(ptr, nbytes), device=torch.device("cuda", device))


class SymmetricBuffer:
    def __init__(self, comm: capi.Comm, nbytes: int, device: int | None = None, register: bool = True):
        self.comm = comm
        self.device = torch.cuda.current_device() if device is None else device
        self.nbytes = int(nbytes)
        self.ptr = capi.mem_alloc(self.nbytes)
        self.win = comm.window_register(self.ptr, self.nbytes) if register else None
        self._bytes = tensor_from_ptr(self.ptr, self.nbytes, self.device)

    def view(self, dtype: torch.dtype, numel: int | None = None, byte_offset: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        if numel is None:
            numel = (self.nbytes - byte_offset) // esz
        return self._bytes[byte_offset:byte_offset + numel * esz].view(dtype)

    def peer_pointer(self, peer: int, offset: int = 0) -> int:
        return capi.window_peer_pointer(self.win, peer, offset)

    def free(self) -> None:
        """Collective (deregistration synchronises the ranks)."""
        if self.ptr is None:
            return
        self._bytes = None
        if self.win is not None:
            self.comm.window_deregister(self.win)
            self.win = None
        capi.mem_free(self.ptr)
        self.ptr = None
