"""Host side of the fused expert-parallel dispatch / combine (``csrc/kernels/ep_dispatch_combine.cu``).

One :class:`EpContext` per engine owns the symmetric buffer and is shared by every MoE layer (layers run
one after the other; the protocol itself orders reuse of the buffer).  ``moe_forward`` replaces the
reference's dispatch -> grouped matmul -> swiglu -> grouped matmul -> combine sequence
(omni/models/common/layers/moe/deepseek_moe.py:370-541)."""
from __future__ import annotations

import ctypes

import torch

from .. import ops
from ..ops import FP8
from ..ops import _native as nat
from .parallel_state import get_parallel_state
from .symmetric_heap import SymmetricBuffer


class EpLayout(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("cap", ctypes.c_int), ("H", ctypes.c_int),
                ("max_slots", ctypes.c_int), ("payload", ctypes.c_int), ("off_recv_x", ctypes.c_longlong), ("off_recv_s", ctypes.c_longlong),
                ("off_recv_meta", ctypes.c_longlong), ("off_recv_cnt", ctypes.c_longlong),
                ("off_recv_flag", ctypes.c_longlong), ("off_comb", ctypes.c_longlong),
                ("off_comb_flag", ctypes.c_longlong), ("off_ctrl", ctypes.c_longlong)]


def _align(x, a=256):
    return (x + a - 1) // a * a


class EpContext:
    def __init__(self, hidden: int, top_k: int, max_tokens: int, wait_ms: float = 2000.0, group=None, payload: str = "fp8"):
        ps = get_parallel_state()
        self.world, self.rank = ps.world_size, ps.rank
        self.H, self.top_k, self.max_tokens = hidden, top_k, max_tokens
        self.cap = max_tokens * top_k                   # worst case: all of a source's pairs land on one rank
        self.max_slots = max_tokens * top_k
        self.wait_ns = int(wait_ms * 1e6)
        W, cap, H = self.world, self.cap, hidden
        off = 0
        self.payload = payload                          # "fp8": e4m3 rows + 1x128 scales; "bf16": rows as they are
        pb = 2 if payload == "bf16" else 1
        lay = EpLayout(world=W, rank=self.rank, cap=cap, H=H, max_slots=self.max_slots, payload=pb)
        lay.off_recv_x = off; off = _align(off + W * cap * H * pb)
        lay.off_recv_s = off; off = _align(off + W * cap * (H // 128) * 4)
        lay.off_recv_meta = off; off = _align(off + W * cap * 16)
        lay.off_recv_cnt = off; off = _align(off + 64 * 4)
        lay.off_recv_flag = off; off = _align(off + 64 * 4)
        lay.off_comb = off; off = _align(off + self.max_slots * H * 2)
        lay.off_comb_flag = off; off = _align(off + 64 * 4)
        lay.off_ctrl = off; off = _align(off + 64 * 4)
        self.layout = lay
        self.buf = SymmetricBuffer(off, group=group)
        self.nbytes = off

    def close(self):
        self.buf.close()

    # ------------------------------------------------------------------ one MoE layer
    def moe_forward(self, layer, x, ids, w, shared, xq=None):
        """x [T,H] bf16, ids/w [T,k] physical expert ids and routing weights -> [T,H].  ``xq`` = (e4m3 rows, K-block-major
        scales) of x, when the caller has them, is sent instead of quantising every (token, expert) pair again."""
        L = nat.lib()
        lay, peers = ctypes.byref(self.layout), self.buf.ptr_array
        T = x.shape[0]
        k = self.top_k
        dev = x.device
        assert T <= self.max_tokens, "batch exceeds the fused EP buffers; the runner must pick the NCCL path"
        st = nat.ptr(nat.status_buffer(dev))
        fp8 = self.payload == "fp8"
        assert fp8 == (layer.quant == "fp8_block"), "payload of the EP buffers does not match the expert weights"
        pre = xq if (fp8 and xq is not None and T > 0) else None
        nat.check_rc(L.omni_ep_dispatch_send(nat.ptr(x), nat.ptr(pre[0]) if pre else None, nat.ptr(pre[1]) if pre else None,
                                             nat.c_int(pre[1].shape[1] if pre else 0), nat.ptr(ids), nat.ptr(w), nat.c_int(T),
                                             nat.c_int(k), nat.c_int(layer.slots_per_rank), lay, peers, st, nat.stream()),
                     "omni_ep_dispatch_send")
        n = self.world * self.cap
        r_ids = torch.empty(n, dtype=torch.int32, device=dev)
        r_w = torch.empty(n, dtype=torch.float32, device=dev)
        r_slot = torch.empty(n, dtype=torch.int32, device=dev)
        nat.check_rc(L.omni_ep_dispatch_recv(lay, peers, nat.ptr(r_ids), nat.ptr(r_w), nat.ptr(r_slot), nat.ptr(None),
                                             ctypes.c_ulonglong(self.wait_ns), st, nat.stream()),
                     "omni_ep_dispatch_recv")
        S = layer.slots_per_rank
        capacity = (n + S * 15 + 15) // 16 * 16
        counts = torch.empty(S, dtype=torch.int32, device=dev)
        pos = torch.empty(n, dtype=torch.int32, device=dev)
        seg_start = torch.empty(S, dtype=torch.int32, device=dev)
        seg_len = torch.empty(S, dtype=torch.int32, device=dev)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        nat.check_rc(L.omni_moe_align(nat.ptr(r_ids), nat.c_int(n), nat.c_int(0), nat.c_int(S), nat.c_int(16),
                                      nat.c_int(capacity), nat.ptr(counts), nat.ptr(pos), nat.ptr(seg_start),
                                      nat.ptr(seg_len), nat.ptr(total), st, nat.stream()), "omni_moe_align")
        # padding rows are never read back (see ops.moe_permute)
        xq = torch.empty(capacity, self.H, dtype=FP8 if fp8 else x.dtype, device=dev)
        xs = torch.empty(self.H // 128, capacity, dtype=torch.float32, device=dev) if fp8 else None
        row_w = torch.empty(capacity, dtype=torch.float32, device=dev)
        row_rank = torch.empty(capacity, dtype=torch.int32, device=dev)
        row_slot = torch.empty(capacity, dtype=torch.int32, device=dev)
        nat.check_rc(L.omni_ep_scatter_q(lay, peers, nat.ptr(r_ids), nat.ptr(pos), nat.ptr(r_w), nat.ptr(r_slot),
                                         nat.ptr(seg_start), nat.ptr(seg_len), nat.ptr(xq), nat.ptr(xs),
                                         nat.c_int(capacity), nat.ptr(row_w), nat.ptr(row_rank), nat.ptr(row_slot),
                                         nat.stream()), "omni_ep_scatter_q")
        t_hint = max(32, (self.max_tokens * k + S - 1) // S if T == 0 else (T * k * 1 + S - 1) // S)
        y = layer.experts(xq, xs, seg_start, seg_len, row_w, t_hint)
        nat.check_rc(L.omni_ep_combine_send(nat.ptr(y), nat.ptr(total), nat.ptr(seg_start), nat.ptr(seg_len),
                                            nat.c_int(S), nat.ptr(row_rank), nat.ptr(row_slot), nat.c_int(capacity),
                                            lay, peers, nat.stream()), "omni_ep_combine_send")
        out = torch.empty(T, self.H, dtype=x.dtype, device=dev)
        layer.join_shared()
        nat.check_rc(L.omni_ep_combine_reduce(lay, peers, nat.ptr(ids), nat.c_int(T), nat.c_int(k), nat.ptr(shared),
                                              nat.ptr(out), ctypes.c_ulonglong(self.wait_ns), st, nat.stream()),
                     "omni_ep_combine_reduce")
        return out
