"""Symmetric device buffers: the same allocation on every rank, peer-addressable.

A :class:`SymmBuffer` is the HBM home of a parameter-server shard.  Each rank
allocates ``numel`` elements, the CUDA IPC handles are exchanged through the
process group (an ``all_gather_object`` over the bootstrap backend), and every
rank ends up with ``ptrs[r]`` = address of rank r's allocation in its own
address space plus a device-resident pointer table that kernels index by owner
rank.  With ``world == 1`` no IPC is involved.

This replaces the reference's socket table (one ``kvclt`` per server,
include/ps.hpp:1249-1265): "connecting to a server" becomes "holding a pointer
to its shard".
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib


class _RawCudaArray:
    """Adapter exposing a raw device pointer through __cuda_array_interface__."""

    def __init__(self, ptr: int, numel: int, typestr: str, owner=None):
        self.__cuda_array_interface__ = {
            "shape": (numel,),
            "typestr": typestr,
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }
        self._owner = owner


_TYPESTR = {
    torch.float32: "<f4",
    torch.int32: "<i4",
    torch.int64: "<i8",
    torch.float64: "<f8",
    torch.uint8: "|u1",
}


class SymmBuffer:
    def __init__(self, numel: int, dtype=torch.float32, group=None, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else
                                   f"cuda:{torch.cuda.current_device()}")
        self.dtype = dtype
        self.numel = int(numel)
        self.itemsize = torch.empty((), dtype=dtype).element_size()
        nbytes = max(256, self.numel * self.itemsize)
        nbytes = (nbytes + 255) // 256 * 256
        self.nbytes = nbytes
        lib = _lib.load()
        with torch.cuda.device(self.device):
            p = ctypes.c_void_p()
            h = (ctypes.c_ubyte * 64)()
            rc = lib.pcl_symm_alloc(nbytes, ctypes.byref(p), h)
            if rc != 0:
                raise RuntimeError(f"pcl_symm_alloc({nbytes}) failed: CUDA error {rc}")
            self._local_ptr = p.value
            self._opened: List[int] = []
            self.ptrs: List[int] = [0] * self.world
            if self.world == 1:
                self.ptrs[0] = self._local_ptr
            else:
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, bytes(h), group=group)
                for r in range(self.world):
                    if r == self.rank:
                        self.ptrs[r] = self._local_ptr
                        continue
                    q = ctypes.c_void_p()
                    hb = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                    rc = lib.pcl_symm_open(hb, ctypes.byref(q))
                    if rc != 0:
                        raise RuntimeError(f"pcl_symm_open(rank {r}) failed: CUDA error {rc}")
                    self.ptrs[r] = q.value
                    self._opened.append(q.value)
            self.local = torch.as_tensor(
                _RawCudaArray(self._local_ptr, max(self.numel, 1), _TYPESTR[dtype], self),
                device=self.device)[: self.numel]
            # pointer table on the device, indexed by owner rank
            self.ptr_table = torch.tensor(self.ptrs, dtype=torch.int64, device=self.device)
        if self.world > 1:
            dist.barrier(group=group)

    def peer_view(self, r: int) -> torch.Tensor:
        """Tensor view of rank r's allocation (peer memory; for tests and debugging)."""
        return torch.as_tensor(
            _RawCudaArray(self.ptrs[r], max(self.numel, 1), _TYPESTR[self.dtype], self),
            device=self.device)[: self.numel]

    def free(self):
        if getattr(self, "_local_ptr", None) is None:
            return
        lib = _lib.load()
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        for q in self._opened:
            lib.pcl_symm_close(q)
        self._opened = []
        if self.world > 1:
            dist.barrier(group=self.group)
        lib.pcl_symm_free(self._local_ptr)
        self._local_ptr = None
        self.local = None
