"""Symmetric device buffers for the fused NVLink kernels.

Each rank allocates one buffer with ``cudaMalloc`` (outside the PyTorch caching allocator so that the
allocation base is what CUDA IPC exports), exchanges the 64-byte IPC handle over the process group and
opens every peer's buffer.  ``peer_ptrs[r]`` is rank r's buffer as seen from this process; kernels index
it with offsets that are identical on all ranks.  The reference gets the same effect from vendor ops that
take a named collective group (omni/models/common/layers/moe/fused_moe/layer.py:265-266)."""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _native as nat


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` wrapper to view raw device memory as a tensor."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    def __init__(self, nbytes: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = (nbytes + 255) // 256 * 256
        L = nat.lib()
        p = ctypes.c_void_p()
        nat.check_rc(L.omni_symm_alloc(ctypes.byref(p), ctypes.c_longlong(self.nbytes)), "omni_symm_alloc")
        self.local_ptr = p.value
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        self._opened = []
        if self.world > 1:
            h = (ctypes.c_ubyte * 64)()
            nat.check_rc(L.omni_symm_get_handle(ctypes.c_void_p(self.local_ptr), h), "omni_symm_get_handle")
            mine = torch.tensor(list(h), dtype=torch.uint8, device="cuda")
            allh = torch.empty(self.world, 64, dtype=torch.uint8, device="cuda")
            dist.all_gather_into_tensor(allh, mine, group=group)
            allh = allh.cpu()
            for r in range(self.world):
                if r == self.rank:
                    continue
                hb = (ctypes.c_ubyte * 64)(*allh[r].tolist())
                q = ctypes.c_void_p()
                nat.check_rc(L.omni_symm_open_handle(hb, ctypes.byref(q)), f"omni_symm_open_handle(rank {r})")
                self.peer_ptrs[r] = q.value
                self._opened.append(q.value)
            dist.barrier(group=group)
        self.ptr_array = (ctypes.c_void_p * 16)(*([ctypes.c_void_p(x) for x in self.peer_ptrs] + [None] * (16 - self.world)))

    def local_tensor(self, offset: int, nbytes: int, dtype=torch.uint8) -> torch.Tensor:
        t = torch.as_tensor(_CudaArray(self.local_ptr + offset, nbytes), device="cuda")
        return t.view(dtype)

    def close(self) -> None:
        L = nat.lib()
        torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        for p in self._opened:
            L.omni_symm_close_handle(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            L.omni_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0


def alloc_ipc_tensor(shape, dtype, device=None) -> torch.Tensor:
    """A zero-filled tensor backed by its own ``cudaMalloc`` allocation, so that its base address can be exported
    with CUDA IPC (tensors from the caching allocator are sub-allocations and cannot)."""
    n = 1
    for d in shape:
        n *= d
    nbytes = n * torch.empty(0, dtype=dtype).element_size()
    p = ctypes.c_void_p()
    nat.check_rc(nat.lib().omni_symm_alloc(ctypes.byref(p), ctypes.c_longlong(max(nbytes, 256))), "omni_symm_alloc")
    t = torch.as_tensor(_CudaArray(p.value, nbytes), device="cuda").view(dtype).view(*shape)
    t._omni_ipc_base = p.value
    return t


def export_ipc_handles(tensors) -> list:
    out = []
    for t in tensors:
        h = (ctypes.c_ubyte * 64)()
        nat.check_rc(nat.lib().omni_symm_get_handle(ctypes.c_void_p(t.data_ptr()), h), "omni_symm_get_handle")
        out.append(bytes(h))
    return out


def open_ipc_handles(handles) -> list:
    ptrs = []
    for hb in handles:
        h = (ctypes.c_ubyte * 64)(*hb)
        q = ctypes.c_void_p()
        nat.check_rc(nat.lib().omni_symm_open_handle(h, ctypes.byref(q)), "omni_symm_open_handle")
        ptrs.append(q.value)
    return ptrs
