"""Expert parallelism over plain collectives (NCCL on GPUs, gloo on CPU ranks): the unfused baseline the
fused NVLink path is measured against, and the path for batches larger than the fused buffers (prefill).
Same data flow as the reference's all-to-all EP (omni/models/common/layers/moe/fused_moe/fused_moe.py:201-383):
sort pairs by destination rank, exchange counts, exchange rows, run the local experts, send rows back,
weighted sum per token."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from .parallel_state import get_parallel_state


def moe_forward_nccl(layer, x, ids, w, shared):
    ps = get_parallel_state()
    g = ps.group("ep")
    W = ps.ep_size
    T, k = ids.shape
    H = x.shape[1]
    S = layer.slots_per_rank
    dev = x.device
    flat_ids = ids.reshape(-1).long()
    valid = flat_ids >= 0
    dest = torch.where(valid, flat_ids // S, torch.full_like(flat_ids, W))      # padding sorts last
    order = torch.argsort(dest, stable=True)
    n_valid = int(valid.sum())
    order = order[:n_valid]
    send_counts = torch.bincount(dest[order], minlength=W)[:W]
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=g.group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    tok = order // k
    send_x = x[tok].contiguous()
    send_e = (flat_ids[order] % S).int().contiguous()
    send_w = w.reshape(-1)[order].float().contiguous()
    n_recv = sum(rc)
    recv_x = torch.empty(n_recv, H, dtype=x.dtype, device=dev)
    recv_e = torch.empty(n_recv, dtype=torch.int32, device=dev)
    recv_w = torch.empty(n_recv, dtype=torch.float32, device=dev)
    dist.all_to_all_single(recv_x, send_x, rc, sc, group=g.group)
    dist.all_to_all_single(recv_e, send_e, rc, sc, group=g.group)
    dist.all_to_all_single(recv_w, send_w, rc, sc, group=g.group)
    # local experts on the received rows (k = 1 from the permutation's point of view)
    perm = ops.moe_permute(recv_x, recv_e.view(-1, 1), recv_w.view(-1, 1), 0, S, quant=layer.quant == "fp8_block")
    t_hint = max(32, (n_recv + S - 1) // S)
    y = layer.experts(perm.x, perm.x_scale, perm.seg_start, perm.seg_len, perm.row_w, t_hint)
    back = y[perm.row_of.long().clamp_min(0)] if n_recv else y[:0]
    ret = torch.empty(n_valid, H, dtype=x.dtype, device=dev)
    dist.all_to_all_single(ret, back.contiguous(), sc, rc, group=g.group)
    out = torch.zeros(T, H, dtype=torch.float32, device=dev)
    out.index_add_(0, tok, ret.float())
    if shared is not None:
        layer.join_shared()
        out += shared.float()
    return out.to(x.dtype)
