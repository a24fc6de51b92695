"""Collectives that reduce inside the NVSwitch (``multimem`` on a multicast mapping), ``csrc/kernels/nvls_collectives.cu``.

The multicast mapping comes from PyTorch's symmetric-memory rendezvous (it creates the multicast object, binds every
rank's allocation and maps it); this module only allocates through it, keeps the addresses and launches the kernels:

  ``all_reduce_``   in place on a view of the workspace: each rank reduces its share with ``multimem.ld_reduce`` and
                    broadcasts the sums with ``multimem.st``
  ``reduce_rows``   reduce-scatter over token rows after a row-parallel GEMM whose partial product was written to the
                    local workspace, with the residual add and RMSNorm in the same kernel

Counterpart of the reference's tensor-parallel all-reduce / reduce-scatter
(omni/adaptors/vllm/distributed/communication_op.py).  A rank that leaves while its memory is bound to a multicast
object faults its peers, so nothing that tests failure handling may create this workspace."""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _native as nat


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


def available(device=None) -> bool:
    """True when the device and the driver offer multicast memory (NVSwitch systems)."""
    try:
        import torch.distributed._symmetric_memory as symm
        from torch._C._distributed_c10d import _SymmetricMemory
        dev = torch.device(device if device is not None else "cuda")
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        return bool(_SymmetricMemory.has_multicast_support(symm.DeviceType.CUDA, idx))
    except Exception:  # noqa: BLE001  (no such API in this build: no NVLS)
        return False


class NvlsWorkspace:
    FLAG_BYTES = 256

    def __init__(self, group, data_bytes: int, wait_ms: float = 2000.0):
        import torch.distributed._symmetric_memory as symm
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert 2 <= self.world <= 8
        self.data_bytes = _align(data_bytes, 4096)
        self.flag_offset = self.data_bytes
        self.wait_ns = int(wait_ms * 1e6)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm.empty(self.data_bytes + self.FLAG_BYTES, dtype=torch.uint8, device=dev)
        self.hdl = symm.rendezvous(self.buf, group=group.group_name if hasattr(group, "group_name") else group)
        self.mc = int(self.hdl.multicast_ptr)
        if not self.mc:
            raise RuntimeError("the symmetric-memory rendezvous returned no multicast mapping (NVLS is not available here)")
        self.peers = [int(p) for p in self.hdl.buffer_ptrs]
        self.buf.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self._peer_arr = (ctypes.c_void_p * 8)(*(self.peers + [None] * (8 - self.world)))

    def view(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        assert nbytes <= self.data_bytes, "the workspace is too small for this tensor"
        return self.buf[:nbytes].view(dtype).view(*shape)

    def all_reduce_(self, numel: int, ctas: int = 0) -> torch.Tensor:
        """Sum over the ranks of the first ``numel`` bf16 elements of the workspace, in place; returns the view."""
        assert numel % 8 == 0
        rc = nat.lib().omni_nvls_allreduce(ctypes.c_void_p(self.mc), ctypes.c_void_p(self.peers[self.rank]), self._peer_arr,
                                           ctypes.c_longlong(self.flag_offset), nat.c_int(self.world), nat.c_int(self.rank),
                                           ctypes.c_longlong(numel), nat.c_int(ctas), ctypes.c_ulonglong(self.wait_ns),
                                           nat.ptr(nat.status_buffer(self.buf.device)), nat.stream())
        nat.check_rc(rc, "omni_nvls_allreduce")
        nat.add_launches(1)
        return self.view((numel,))

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Convenience form for a tensor that lives elsewhere: copy in, reduce, copy out."""
        assert x.dtype == torch.bfloat16 and x.is_contiguous()
        v = self.view(tuple(x.shape))
        v.copy_(x)
        self.all_reduce_(x.numel())
        return v.clone()

    def reduce_rows(self, total_rows: int, n: int, residual=None, norm_weight=None, eps: float = 1e-6):
        """The workspace holds this rank's partial [total_rows, n]; returns the summed rows of this rank's block
        (+ residual), and their RMSNorm when ``norm_weight`` is given."""
        assert total_rows % self.world == 0 and n % 8 == 0
        rpr = total_rows // self.world
        dev = self.buf.device
        out = torch.empty(rpr, n, dtype=torch.bfloat16, device=dev)
        normed = torch.empty_like(out) if norm_weight is not None else None
        rc = nat.lib().omni_nvls_reduce_rows(ctypes.c_void_p(self.mc), ctypes.c_void_p(self.peers[self.rank]), self._peer_arr,
                                             ctypes.c_longlong(self.flag_offset), nat.c_int(self.world), nat.c_int(self.rank),
                                             nat.c_int(rpr), nat.c_int(n), nat.ptr(residual), nat.ptr(out), nat.ptr(norm_weight),
                                             nat.ptr(normed), nat.c_float(eps), ctypes.c_ulonglong(self.wait_ns),
                                             nat.ptr(nat.status_buffer(dev)), nat.stream())
        nat.check_rc(rc, "omni_nvls_reduce_rows")
        nat.add_launches(1)
        return (out, normed) if norm_weight is not None else out
