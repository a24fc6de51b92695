"""Tensor-parallel attention block with the collectives fused into the GEMMs (one node, NVLink peer memory).

Between layers the hidden states are sharded by token rows (rank r owns rows ``[r*rpr, (r+1)*rpr)``), which is
what the expert-parallel MoE wants.  The attention block is sharded by heads, so it needs all rows:

* ``allgather_gemm``       all-gather of the row blocks fused into the first projection (q_a / kv_a, or the first
                           MLP GEMM): every rank pushes its block into all gather buffers, and the GEMM on each
                           rank waits per source block inside its TMA producer, starting with its own rows.
* ``gemm_reduce_scatter``  the row-parallel o_proj GEMM whose epilogue writes each partial row into the receive
                           slab of the rank that owns the row; a small kernel then adds the slabs (and, if asked,
                           the residual and the next RMSNorm).

The kernels are ``gemm_tokmajor_sm100.cu`` and ``tp_fused.cu``.  ``TpNcclBaseline`` does the same with NCCL
collectives around plain GEMMs; tests compare the two, and CPU (gloo) runs use the baseline.
Reference behaviour: omni/models/common/layers/attention/deepseek_mla.py:437-470 (all_gather before the q/kv
projections, reduce_scatter after o_proj) and omni/models/common/layers/linear.py:139-199 (row/column parallel
linears with explicit collectives).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _native as nat
from ..ops.gemm import FP8, TmCollective, _tm2
from .symmetric_heap import SymmetricBuffer


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class TpFusedContext:
    """Symmetric buffers + round counters for the fused tensor-parallel GEMMs of one process group.

    Every rank must issue the same sequence of calls.  The gather buffer and the reduce-scatter slab are single
    buffers: ``allgather_gemm`` and ``gemm_reduce_scatter`` calls must alternate (as they do in a layer: all-gather
    before the attention block, reduce-scatter after it), because a reduce-scatter only completes on a rank when every
    rank has finished the GEMM that read the previous gather, and the next push can only overtake a rank that has
    finished its slab reduce.  ``all_gather_rows`` and ``all_reduce`` use their own buffers with two halves selected by
    a round counter in device memory, so they may be called at any point of the sequence.  All counters and flags
    live in device memory and advance inside the kernels: the calls can be captured in a CUDA graph and replayed."""

    def __init__(self, group, max_tokens: int, max_k_bytes: int, max_n: int, wait_ms: float = 2000.0, nvls: bool = False):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert 2 <= self.world <= 8
        self.max_tokens = _align(max_tokens, 128 * self.world) if max_tokens >= 128 * self.world else \
            (max_tokens + self.world - 1) // self.world * self.world
        self.max_rpr = self.max_tokens // self.world
        self.max_k_bytes = _align(max_k_bytes, 16)
        self.max_n = _align(max_n, 8)
        self.wait_ns = int(wait_ms * 1e6)
        # layout (identical on every rank)
        off = 0
        self.off_gather = off; off = _align(off + self.max_tokens * self.max_k_bytes)
        self.off_gather_scale = off; off = _align(off + (self.max_k_bytes // 128 + 1) * self.max_tokens * 4)
        self.off_slab = off; off = _align(off + self.world * self.max_rpr * self.max_n * 2)
        self.off_ag_flag = off; off = _align(off + 64)
        self.off_rs_flag = off; off = _align(off + 64)
        self.off_fin = off; self.fin_half = _align(self.max_tokens * self.max_k_bytes); off = _align(off + 2 * self.fin_half)
        self.off_fin_flag = off; off = _align(off + 64)
        self.ar_rows = min(self.max_tokens, 1024)         # all-reduce is for decode-sized messages
        self.off_ar = off; self.ar_half = _align(self.world * self.ar_rows * self.max_n * 2); off = _align(off + 2 * self.ar_half)
        self.off_ar_flag = off; off = _align(off + 64)
        self.off_ctrl = off; off = _align(off + 64)     # [0] ag round, [1] ag done, [2] rs round, [3] rs done, [4] final round, [5] final done, [6] ar round, [7] ar done
        self.buf = SymmetricBuffer(off, group)
        self.buf.local_tensor(0, off).zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        lp = self.buf.local_ptr
        self._ag_round = lp + self.off_ctrl
        self._ag_done = lp + self.off_ctrl + 4
        self._rs_round = lp + self.off_ctrl + 8
        self._rs_done = lp + self.off_ctrl + 12
        self._fin_round = lp + self.off_ctrl + 16
        self._fin_done = lp + self.off_ctrl + 20
        self._ar_round = lp + self.off_ctrl + 24
        self._ar_done = lp + self.off_ctrl + 28
        # in-switch reduction (multimem) for the two reducing collectives: the row-parallel GEMM then writes its
        # partial product to local memory and every rank pulls the sums of its rows through the NVSwitch, instead of
        # every rank storing its partial rows into the owner's slab
        self.nvls = None
        if nvls:
            from .nvls import NvlsWorkspace
            self.nvls = NvlsWorkspace(group, self.max_tokens * self.max_n * 2, wait_ms)

    # ------------------------------------------------------------------ helpers
    def rows_per_rank(self, total_rows: int) -> int:
        assert total_rows % self.world == 0, "token rows are padded to a multiple of the TP world size"
        return total_rows // self.world

    def _peer(self, r: int, off: int) -> int:
        return self.buf.peer_ptrs[r] + off

    # ------------------------------------------------------------------ all-gather + GEMM
    def allgather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, total_rows: int, w_scale=None,
                       x_scale_shard=None, epi: str = "store", out_dtype=torch.bfloat16):
        """``gemm(all_gather(x_shard), w)`` with the gather overlapped.  x_shard: [rpr, K] bf16, or e4m3 with
        ``x_scale_shard`` [K/128, rpr] (K-block major).  Returns ([total_rows, n_out], gathered x view[, scales])."""
        rpr = self.rows_per_rank(total_rows)
        assert x_shard.shape[0] == rpr and x_shard.is_contiguous()
        K = x_shard.shape[1]
        esz = x_shard.element_size()
        row_bytes = K * esz
        assert row_bytes % 16 == 0 and row_bytes <= self.max_k_bytes and total_rows <= self.max_tokens
        L = nat.lib()
        gather = (ctypes.c_void_p * 8)(*[self._peer(r, self.off_gather) for r in range(self.world)] + [None] * (8 - self.world))
        flags = (ctypes.c_void_p * 8)(*[self._peer(r, self.off_ag_flag + 4 * self.rank) for r in range(self.world)]
                                      + [None] * (8 - self.world))
        fp8 = x_shard.dtype == FP8
        xs_full = None
        if fp8:
            # activation scales travel as one more (small) gather: [K/128, total_rows], this rank's columns
            kb = x_scale_shard.shape[0]
            assert x_scale_shard.shape[1] == rpr and rpr % 4 == 0
            xs_full = self.buf.local_tensor(self.off_gather_scale, kb * total_rows * 4, torch.float32).view(kb, total_rows)
            # scales are a few KB; they go in front of the row push on the same stream and are covered by its flag
            sc = (ctypes.c_void_p * 8)(*[self._peer(r, self.off_gather_scale) for r in range(self.world)]
                                       + [None] * (8 - self.world))
            xs_c = x_scale_shard.contiguous()
            rc = L.omni_ag_push(nat.ptr(xs_c), nat.c_int(kb), nat.c_int(rpr * 4), ctypes.c_longlong(total_rows * 4),
                                ctypes.c_longlong(self.rank * rpr * 4), ctypes.c_longlong(0), nat.c_int(self.world),
                                nat.c_int(self.rank), nat.c_int(0), sc, flags, None, None, nat.stream())
            nat.check_rc(rc, "omni_ag_push(scales)")
            nat.add_launches(1)
        rc = L.omni_ag_push(nat.ptr(x_shard), nat.c_int(rpr), nat.c_int(row_bytes), ctypes.c_longlong(row_bytes),
                            ctypes.c_longlong(self.rank * rpr * row_bytes), ctypes.c_longlong(0), nat.c_int(self.world),
                            nat.c_int(self.rank), nat.c_int(1), gather, flags, ctypes.c_void_p(self._ag_round), ctypes.c_void_p(self._ag_done),
                            nat.stream())
        nat.check_rc(rc, "omni_ag_push")
        nat.add_launches(1)
        x_full = self.buf.local_tensor(self.off_gather, total_rows * row_bytes, x_shard.dtype).view(total_rows, K)
        coll = TmCollective()
        coll.ag_world, coll.ag_rank, coll.ag_rows_per_rank = self.world, self.rank, rpr
        coll.ag_flag = self.buf.local_ptr + self.off_ag_flag
        coll.ag_epoch = self._ag_round
        coll.ag_wait_ns = self.wait_ns
        e = {"store": 0, "swiglu": 1, "swiglu_quant": 2}[epi]
        if w.dim() == 2:
            w = w.unsqueeze(0)
        n_w = w.shape[1]
        n_out = n_w if e == 0 else n_w // 2
        if e == 2:
            out = torch.empty(total_rows, n_out, dtype=FP8, device=x_shard.device)
            out_scale = torch.zeros(n_out // 128, max(4, (total_rows + 3) // 4 * 4), dtype=torch.float32, device=x_shard.device)
        else:
            out = torch.empty(total_rows, n_out, dtype=out_dtype if e == 0 else torch.bfloat16, device=x_shard.device)
            out_scale = None
        _tm2(1 if fp8 else 0, e, w, x_full, out, 1, n_out, K, total_rows, None, None, w_scale, xs_full,
             1 if out.dtype == torch.float32 else 0, out_scale, None, coll=coll)
        if e == 2:
            return (out, out_scale), x_full, xs_full
        return out, x_full, xs_full

    # ------------------------------------------------------------------ plain all-gather of rows
    def all_gather_rows(self, x_shard: torch.Tensor, total_rows: int) -> torch.Tensor:
        """[rpr, K] on every rank -> [total_rows, K] on every rank, through peer stores and flags (no library call, so it
        can sit inside a captured CUDA graph).  Used for the final hidden states, which every rank samples from."""
        rpr = self.rows_per_rank(total_rows)
        assert x_shard.shape[0] == rpr and x_shard.is_contiguous()
        row_bytes = x_shard.shape[1] * x_shard.element_size()
        assert row_bytes % 16 == 0 and row_bytes <= self.max_k_bytes and total_rows <= self.max_tokens
        L = nat.lib()
        gather = (ctypes.c_void_p * 8)(*[self._peer(r, self.off_fin) for r in range(self.world)] + [None] * (8 - self.world))
        flags = (ctypes.c_void_p * 8)(*[self._peer(r, self.off_fin_flag + 4 * self.rank) for r in range(self.world)]
                                      + [None] * (8 - self.world))
        rc = L.omni_ag_push(nat.ptr(x_shard), nat.c_int(rpr), nat.c_int(row_bytes), ctypes.c_longlong(row_bytes),
                            ctypes.c_longlong(self.rank * rpr * row_bytes), ctypes.c_longlong(self.fin_half),
                            nat.c_int(self.world), nat.c_int(self.rank), nat.c_int(1), gather, flags,
                            ctypes.c_void_p(self._fin_round), ctypes.c_void_p(self._fin_done), nat.stream())
        nat.check_rc(rc, "omni_ag_push(final)")
        out = torch.empty(total_rows, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        rc = L.omni_ag_collect(ctypes.c_void_p(self.buf.local_ptr + self.off_fin), ctypes.c_longlong(self.fin_half), nat.ptr(out),
                               ctypes.c_longlong(total_rows * row_bytes), nat.c_int(self.world),
                               ctypes.c_void_p(self.buf.local_ptr + self.off_fin_flag), ctypes.c_void_p(self._fin_round),
                               ctypes.c_ulonglong(self.wait_ns), nat.ptr(nat.status_buffer(x_shard.device)), nat.stream())
        nat.check_rc(rc, "omni_ag_collect")
        nat.add_launches(2)
        return out

    # ------------------------------------------------------------------ one-shot all-reduce
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of ``x`` [rows, n] (bf16) over the ranks, for decode-sized messages: every rank stores its rows into
        its slot on every rank (two halves used in turn, chosen by the round counter in device memory), then each
        rank adds the slots in fp32.  One NVLink crossing, no library call."""
        rows, n = x.shape
        if self.nvls is not None:
            return self.nvls.all_reduce(x)
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and n % 8 == 0 and n <= self.max_n and rows <= self.ar_rows
        L = nat.lib()
        slot_bytes = self.ar_rows * self.max_n * 2
        gather = (ctypes.c_void_p * 8)(*[self._peer(r, self.off_ar) for r in range(self.world)] + [None] * (8 - self.world))
        flags = (ctypes.c_void_p * 8)(*[self._peer(r, self.off_ar_flag + 4 * self.rank) for r in range(self.world)]
                                      + [None] * (8 - self.world))
        rc = L.omni_ag_push(nat.ptr(x), nat.c_int(rows), nat.c_int(n * 2), ctypes.c_longlong(n * 2),
                            ctypes.c_longlong(self.rank * slot_bytes), ctypes.c_longlong(self.ar_half), nat.c_int(self.world),
                            nat.c_int(self.rank), nat.c_int(1), gather, flags, ctypes.c_void_p(self._ar_round),
                            ctypes.c_void_p(self._ar_done), nat.stream())
        nat.check_rc(rc, "omni_ag_push(all_reduce)")
        out = torch.empty_like(x)
        rc = L.omni_rs_reduce2(ctypes.c_void_p(self.buf.local_ptr + self.off_ar), ctypes.c_longlong(self.ar_half),
                               nat.c_int(self.world), nat.c_int(rows), nat.c_int(n), nat.c_int(n),
                               ctypes.c_longlong(slot_bytes // 2), ctypes.c_void_p(self.buf.local_ptr + self.off_ar_flag),
                               ctypes.c_void_p(self._ar_round), ctypes.c_ulonglong(self.wait_ns), None, nat.ptr(out), None, None,
                               nat.c_float(0.0), nat.ptr(nat.status_buffer(x.device)), nat.stream())
        nat.check_rc(rc, "omni_rs_reduce2")
        nat.add_launches(2)
        return out

    # ------------------------------------------------------------------ GEMM + reduce-scatter
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, *, w_scale=None, x_scale=None, residual=None,
                            norm_weight=None, eps: float = 1e-6):
        """``reduce_scatter(gemm(x, w))`` over token rows: x [T, K_local] (this rank's heads), w [N, K_local].
        Returns this rank's rows of the sum (plus ``residual`` [rpr, N] if given) and, with ``norm_weight``, their
        RMSNorm as a second tensor."""
        T = x.shape[0]
        rpr = self.rows_per_rank(T)
        if w.dim() == 2:
            w = w.unsqueeze(0)
        N, K = w.shape[1], w.shape[2]
        assert N <= self.max_n and N % 8 == 0 and rpr <= self.max_rpr
        if self.nvls is not None:
            fp8 = x.dtype == FP8
            part = self.nvls.view((T, N))
            _tm2(1 if fp8 else 0, 0, w, x, part, 1, N, K, T, None, None, w_scale, x_scale, 0, None, None, out_ld=N)
            return self.nvls.reduce_rows(T, N, residual=residual, norm_weight=norm_weight, eps=eps)
        coll = TmCollective()
        coll.rs_world, coll.rs_rank, coll.rs_rows_per_rank = self.world, self.rank, rpr
        for d in range(self.world):
            coll.rs_out[d] = self._peer(d, self.off_slab)
            coll.rs_flag[d] = self._peer(d, self.off_rs_flag + 4 * self.rank)
        coll.rs_done = self._rs_done
        coll.rs_epoch = self._rs_round
        fp8 = x.dtype == FP8
        dummy = self.buf.local_tensor(self.off_slab, 16, torch.bfloat16)
        _tm2(1 if fp8 else 0, 0, w, x, dummy, 1, N, K, T, None, None, w_scale, x_scale, 0, None, None, out_ld=N, coll=coll)
        out = torch.empty(rpr, N, dtype=torch.bfloat16, device=x.device)
        normed = torch.empty_like(out) if norm_weight is not None else None
        rc = nat.lib().omni_rs_reduce(
            ctypes.c_void_p(self.buf.local_ptr + self.off_slab), nat.c_int(self.world), nat.c_int(rpr), nat.c_int(N),
            nat.c_int(N), ctypes.c_longlong(rpr * N), ctypes.c_void_p(self.buf.local_ptr + self.off_rs_flag),
            ctypes.c_void_p(self._rs_round), ctypes.c_ulonglong(self.wait_ns), nat.ptr(residual), nat.ptr(out),
            nat.ptr(norm_weight), nat.ptr(normed), nat.c_float(eps), nat.ptr(nat.status_buffer(x.device)), nat.stream())
        nat.check_rc(rc, "omni_rs_reduce")
        nat.add_launches(1)
        return (out, normed) if norm_weight is not None else out

    def close(self):
        self.buf.close()


class TpNcclBaseline:
    """Same interface with library collectives around plain GEMMs (the comparison baseline; also the CPU path)."""

    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def rows_per_rank(self, total_rows: int) -> int:
        assert total_rows % self.world == 0
        return total_rows // self.world

    def allgather_gemm(self, x_shard, w, *, total_rows, w_scale=None, x_scale_shard=None, epi="store", out_dtype=None):
        rpr = self.rows_per_rank(total_rows)
        if out_dtype is None:      # the model's activation type
            out_dtype = torch.bfloat16 if x_shard.dtype == FP8 else x_shard.dtype
        if x_shard.dtype == FP8:
            xb = torch.empty(total_rows, x_shard.shape[1], dtype=torch.uint8, device=x_shard.device)
            dist.all_gather_into_tensor(xb, x_shard.view(torch.uint8).contiguous(), group=self.group)
            x_full = xb.view(FP8)
            parts = [torch.empty_like(x_scale_shard) for _ in range(self.world)]
            dist.all_gather(parts, x_scale_shard.contiguous(), group=self.group)
            xs_full = torch.cat(parts, dim=1).contiguous()
        else:
            x_full = torch.empty(total_rows, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
            dist.all_gather_into_tensor(x_full, x_shard.contiguous(), group=self.group)
            xs_full = None
        out = ops.gemm(x_full, w, w_scale=w_scale, x_scale=xs_full, epi=epi, out_dtype=out_dtype)
        return out, x_full, xs_full

    def all_gather_rows(self, x_shard, total_rows):
        out = torch.empty(total_rows, x_shard.shape[1], dtype=x_shard.dtype, device=x_shard.device)
        dist.all_gather_into_tensor(out, x_shard.contiguous(), group=self.group)
        return out

    def all_reduce(self, x):
        y = x.float()
        dist.all_reduce(y, group=self.group)
        return y.to(x.dtype)

    def gemm_reduce_scatter(self, x, w, *, w_scale=None, x_scale=None, residual=None, norm_weight=None, eps=1e-6):
        T = x.shape[0]
        rpr = self.rows_per_rank(T)
        part = ops.gemm(x, w, w_scale=w_scale, x_scale=x_scale, out_dtype=torch.float32)   # partial sums stay fp32
        if dist.get_backend(self.group) == "gloo":
            full = part.float()
            dist.all_reduce(full, group=self.group)
            out = full[self.rank * rpr:(self.rank + 1) * rpr]
        else:
            out32 = torch.empty(rpr, part.shape[1], dtype=torch.float32, device=x.device)
            dist.reduce_scatter_tensor(out32, part.float().contiguous(), group=self.group)
            out = out32
        if residual is not None:
            out = out + residual.float()
        # the model's activation type: bf16 on the GPU; fp32 models (CPU test sizes) keep fp32 rows
        out = out.to(residual.dtype if residual is not None else (torch.bfloat16 if x.dtype == FP8 else x.dtype))
        if norm_weight is not None:
            return out, ops.rmsnorm(out, norm_weight, eps)
        return out
