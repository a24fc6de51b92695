"""Block transfer back ends of the PD connector.

``push_blocks`` copies cache blocks ``src_blocks`` of every layer tensor of the prefill instance into blocks
``dst_blocks`` of the decode instance.  On GPUs the destination tensors are peer memory (the decode process's
cache opened through CUDA IPC) and the copy is ``csrc/kernels/kv_push.cu``; on CPU (mock / tests) both sides are
ordinary tensors and the copy is an index assignment."""
from __future__ import annotations

import ctypes

import torch

from ...ops import _native as nat


def flatten_cache(kv_caches) -> list:
    """Layer caches (tensor, or (k, v) pair) -> flat list of tensors [blocks, ...]."""
    out = []
    for c in kv_caches:
        if isinstance(c, (tuple, list)):
            out.extend(c)
        else:
            out.append(c)
    return out


def push_blocks_torch(src_tensors, dst_tensors, src_blocks, dst_blocks) -> None:
    si = torch.as_tensor(src_blocks, dtype=torch.long)
    di = torch.as_tensor(dst_blocks, dtype=torch.long)
    for s, d in zip(src_tensors, dst_tensors):
        d[di.to(d.device)] = s[si.to(s.device)].to(d.device)


class PeerCacheView:
    """Raw device pointers of a (remote) cache: one per layer tensor, plus block geometry."""

    def __init__(self, ptrs: list, block_bytes: int, num_blocks: int):
        self.ptrs, self.block_bytes, self.num_blocks = ptrs, block_bytes, num_blocks


_push_streams: dict = {}


def _push_stream(dev) -> "torch.cuda.Stream":
    """One high-priority, non-blocking stream per device for KV pushes: a push must not queue behind the prefill that
    the producer is running on its compute stream (hundreds of milliseconds for a long prompt), nor order itself
    against it; the blocks it reads were complete before the request's first token left the producer."""
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _push_streams:
        _lo, hi = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, "priority_range") else (0, -1)
        _push_streams[key] = torch.cuda.Stream(device=dev, priority=hi)
    return _push_streams[key]


def push_blocks_cuda(src_tensors, dst_view: PeerCacheView, src_blocks, dst_blocks, stream=None) -> None:
    dev = src_tensors[0].device
    n_t = len(src_tensors)
    assert n_t == len(dst_view.ptrs)
    bb = src_tensors[0][0].numel() * src_tensors[0].element_size()
    assert bb == dst_view.block_bytes, "prefill and decode caches must use the same block geometry"
    st = stream if stream is not None else _push_stream(dev)
    with torch.cuda.device(dev), torch.cuda.stream(st):
        # one pinned staging tensor for the four index arrays: a single asynchronous copy on the push stream
        host = torch.tensor([t.data_ptr() for t in src_tensors] + list(dst_view.ptrs) + list(src_blocks) + list(dst_blocks),
                            dtype=torch.int64).pin_memory()
        devt = host.to(dev, non_blocking=True)
        nb = len(src_blocks)
        src_ptrs, dst_ptrs, sb, db = devt[:n_t], devt[n_t:2 * n_t], devt[2 * n_t:2 * n_t + nb], devt[2 * n_t + nb:]
        rc = nat.lib().omni_kv_push(nat.ptr(src_ptrs), nat.ptr(dst_ptrs), nat.ptr(sb), nat.ptr(db),
                                    ctypes.c_longlong(bb), ctypes.c_longlong(src_tensors[0].shape[0]),
                                    ctypes.c_longlong(dst_view.num_blocks), nat.c_int(n_t), nat.c_int(len(src_blocks)),
                                    nat.ptr(None), nat.ptr(nat.status_buffer(dev)), ctypes.c_void_p(st.cuda_stream))
    nat.check_rc(rc, "omni_kv_push")
    st.synchronize()       # the "done" control message may only leave after the data is on the peer
