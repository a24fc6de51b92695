"""MoE routing and local token permutation (router top-k, align, scatter, combine).

CUDA tensors run ``csrc/kernels/moe_route.cu``.  The references follow the reference project's
``grouped_topk`` / ``fused_topk`` (omni/models/common/layers/moe/fused_moe/fused_moe.py:24-84) and the
device-op routing of DeepSeek-V3 (omni/models/common/layers/moe/fused_moe/layer.py:341-351).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native as nat
from .gemm import FP8, quant_fp8_block_ref


def router_topk_ref(logits, top_k, *, mode="softmax", bias=None, n_group=1, topk_group=1, group_mode="max",
                    renorm=False, scale=1.0, selector=None, forced_balance=False):
    T, E = logits.shape
    if forced_balance:
        ids = (torch.arange(T * top_k, device=logits.device).view(T, top_k)) % E
        w = torch.full((T, top_k), scale / top_k, dtype=torch.float32, device=logits.device)
    else:
        lf = logits.float()
        scores = torch.softmax(lf, dim=-1) if mode == "softmax" else torch.sigmoid(lf)
        sel = scores + bias.float() if bias is not None else scores.clone()
        if n_group > 1:
            g = sel.view(T, n_group, E // n_group)
            gs = g.topk(2, dim=-1).values.sum(-1) if group_mode == "top2sum" else g.max(-1).values
            keep = torch.zeros_like(gs, dtype=torch.bool)
            keep.scatter_(1, gs.topk(topk_group, dim=-1).indices, True)
            sel = sel.masked_fill(~keep.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E), float("-inf"))
        ids = sel.topk(top_k, dim=-1).indices
        w = scores.gather(1, ids)
        if renorm:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * scale
    if selector is not None:
        ids = selector.long()[ids]
    return ids.int(), w.float()


def router_topk(logits, top_k, *, mode="softmax", bias=None, n_group=1, topk_group=1, group_mode="max",
                renorm=False, scale=1.0, selector=None, counts=None, forced_balance=False, num_valid=None):
    """logits fp32 [T, E] -> (physical expert ids int32 [T,k], weights fp32 [T,k]).

    ``selector`` int32 [E] maps logical to physical expert ids (OmniPlacement); ``counts`` int64
    [n_physical] receives the activation histogram; ``num_valid`` (device int32 scalar) marks rows at or
    beyond it as padding (ids = -1)."""
    if not logits.is_cuda:
        ids, w = router_topk_ref(logits, top_k, mode=mode, bias=bias, n_group=n_group, topk_group=topk_group,
                                 group_mode=group_mode, renorm=renorm, scale=scale, selector=selector,
                                 forced_balance=forced_balance)
        if counts is not None:
            counts += torch.bincount(ids.flatten().long(), minlength=counts.numel()).to(counts.dtype)
        return ids, w
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    rc = nat.lib().omni_router_topk(
        nat.ptr(logits), nat.ptr(bias), nat.c_int(T), nat.c_int(E), nat.c_int(0 if mode == "softmax" else 1),
        nat.c_int(n_group), nat.c_int(topk_group), nat.c_int(1 if group_mode == "top2sum" else 0), nat.c_int(top_k),
        nat.c_int(1 if renorm else 0), nat.c_float(scale), nat.ptr(selector), nat.ptr(counts),
        nat.c_int(counts.numel() if counts is not None else 0), nat.c_int(1 if forced_balance else 0), nat.ptr(num_valid),
        nat.ptr(ids), nat.ptr(w), nat.ptr(nat.status_buffer(logits.device)), nat.stream())
    nat.check_rc(rc, "omni_router_topk")
    return ids, w


@dataclass
class MoePermutation:
    """Expert-sorted view of a token batch for one rank's experts [e_lo, e_lo + e_local)."""
    x: torch.Tensor            # [capacity, H] bf16 or e4m3
    x_scale: torch.Tensor | None   # [H/128, capacity] when quantised
    seg_start: torch.Tensor    # int32 [e_local]
    seg_len: torch.Tensor      # int32 [e_local]
    row_of: torch.Tensor       # int32 [T*k]  row of each (token, k) or -1
    row_w: torch.Tensor        # fp32 [capacity] routing weight of each row
    total_rows: torch.Tensor   # int32 [1]


def moe_permute_ref(x, ids, w, e_lo, e_local, quant=False, align=16, capacity=None):
    T, k = ids.shape
    H = x.shape[1]
    flat = ids.flatten().long() - e_lo
    local = (flat >= 0) & (flat < e_local)
    counts = torch.bincount(flat[local], minlength=e_local)
    padded = (counts + align - 1) // align * align
    seg_start = torch.cumsum(padded, 0) - padded
    cap = capacity if capacity is not None else max(int(padded.sum()), align)
    xp = torch.zeros(cap, H, dtype=x.dtype, device=x.device)
    row_of = torch.full((T * k,), -1, dtype=torch.int32, device=x.device)
    row_w = torch.zeros(cap, dtype=torch.float32, device=x.device)
    fill = torch.zeros(e_local, dtype=torch.long)
    for i in range(T * k):
        if local[i]:
            e = int(flat[i])
            r = int(seg_start[e] + fill[e])
            fill[e] += 1
            xp[r] = x[i // k]
            row_of[i] = r
            row_w[r] = w.flatten()[i]
    xs = None
    if quant:
        xp, xs = quant_fp8_block_ref(xp, ld=cap)
    return MoePermutation(xp, xs, seg_start.int(), counts.int(), row_of, row_w,
                          torch.tensor([int(padded.sum())], dtype=torch.int32))


def moe_permute(x, ids, w, e_lo, e_local, quant=False, align=16, capacity=None, xq_in=None):
    """Sort token rows by local expert.  ``capacity`` bounds the permuted buffer (default: worst case).  With ``quant`` the
    rows come out as e4m3 + scales; ``xq_in`` = (e4m3 rows, K-block-major scales) of ``x`` lets them be copied instead of
    quantised once per routed expert."""
    if not x.is_cuda:
        return moe_permute_ref(x, ids, w, e_lo, e_local, quant, align, capacity)
    T, k = ids.shape
    H = x.shape[1]
    n = T * k
    if capacity is None:
        capacity = (n + e_local * (align - 1) + align - 1) // align * align
    dev = x.device
    L = nat.lib()
    counts = torch.empty(e_local, dtype=torch.int32, device=dev)
    pos = torch.empty(n, dtype=torch.int32, device=dev)
    seg_start = torch.empty(e_local, dtype=torch.int32, device=dev)
    seg_len = torch.empty(e_local, dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=torch.int32, device=dev)
    rc = L.omni_moe_align(nat.ptr(ids), nat.c_int(n), nat.c_int(e_lo), nat.c_int(e_local), nat.c_int(align),
                          nat.c_int(capacity), nat.ptr(counts), nat.ptr(pos), nat.ptr(seg_start), nat.ptr(seg_len),
                          nat.ptr(total), nat.ptr(nat.status_buffer(dev)), nat.stream())
    nat.check_rc(rc, "omni_moe_align")
    row_of = torch.empty(n, dtype=torch.int32, device=dev)
    # Rows between a segment's length and its aligned end are never written and never read back: the GEMMs compute a
    # token row only from that row's own inputs and store valid rows only, so the buffers need no zero fill (32 MB per
    # layer at decode sizes).
    row_w = torch.empty(capacity, dtype=torch.float32, device=dev)
    if quant:
        xq = torch.empty(capacity, H, dtype=FP8, device=dev)
        xs = torch.empty(H // 128, capacity, dtype=torch.float32, device=dev)
        xp = None
    else:
        xp = torch.empty(capacity, H, dtype=x.dtype, device=dev)
        xq = xs = None
    if quant and xq_in is not None:
        rc = L.omni_moe_scatter_q8(nat.ptr(xq_in[0]), nat.ptr(xq_in[1]), nat.c_int(xq_in[1].shape[1]), nat.c_int(H),
                                   nat.ptr(ids), nat.ptr(w), nat.ptr(pos), nat.c_int(n), nat.c_int(k), nat.c_int(e_lo),
                                   nat.ptr(seg_start), nat.ptr(seg_len), nat.ptr(xq), nat.ptr(xs), nat.c_int(capacity),
                                   nat.ptr(row_of), nat.ptr(row_w), nat.ptr(None), nat.stream())
        nat.check_rc(rc, "omni_moe_scatter_q8")
        return MoePermutation(xq, xs, seg_start, seg_len, row_of, row_w, total)
    rc = L.omni_moe_scatter(nat.ptr(x), nat.c_int(H), nat.ptr(ids), nat.ptr(w), nat.ptr(pos), nat.c_int(n),
                            nat.c_int(k), nat.c_int(e_lo), nat.ptr(seg_start), nat.ptr(seg_len), nat.ptr(xp),
                            nat.ptr(xq), nat.ptr(xs), nat.c_int(capacity), nat.ptr(row_of), nat.ptr(row_w),
                            nat.ptr(None), nat.stream())
    nat.check_rc(rc, "omni_moe_scatter")
    return MoePermutation(xq if quant else xp, xs, seg_start, seg_len, row_of, row_w, total)


def moe_combine_ref(y, row_of, T, top_k, w=None, shared=None):
    H = y.shape[1]
    out = torch.zeros(T, H, dtype=torch.float32, device=y.device)
    ro = row_of.view(T, top_k).long()
    for k in range(top_k):
        ok = ro[:, k] >= 0
        contrib = y[ro[:, k].clamp_min(0)].float()
        if w is not None:
            contrib = contrib * w.view(T, top_k)[:, k:k + 1]
        out += contrib * ok.unsqueeze(-1)
    if shared is not None:
        out += shared.float()
    return out.to(y.dtype)


def moe_combine(y, row_of, T, top_k, w=None, shared=None):
    """out[t] = sum_k (w[t,k]) * y[row_of[t,k]] (+ shared[t]); summation order over k is fixed."""
    if not y.is_cuda:
        return moe_combine_ref(y, row_of, T, top_k, w, shared)
    H = y.shape[1]
    out = torch.empty(T, H, dtype=y.dtype, device=y.device)
    rc = nat.lib().omni_moe_combine(nat.ptr(y), nat.c_int(H), nat.ptr(row_of), nat.ptr(w), nat.c_int(T),
                                    nat.c_int(top_k), nat.ptr(shared), nat.ptr(out), nat.stream())
    nat.check_rc(rc, "omni_moe_combine")
    return out
