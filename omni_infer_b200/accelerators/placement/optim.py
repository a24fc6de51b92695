"""Token-level routing optimizers of the reference's ``omni_planner/optim`` package (configured through
``Optimizers:`` in its config.yaml; the reference itself currently bypasses them, omni_planner.py:88-91).
Kept as small pure-PyTorch post-processors of (token, topk ids, topk weights)."""
from __future__ import annotations

import torch


class Optimizer:
    def optimize(self, layer: int, tokens, topk_ids, topk_weights, cluster_status=None):
        return tokens, topk_ids, topk_weights


class AdaRouter(Optimizer):
    """Drops low-weight experts: keeps expert j of a token while its weight >= threshold * the token's best weight
    (``threshold``) or the top ``k_keep`` ones (``topk``)."""

    def __init__(self, threshold: float = 0.0, k_keep: int = 0, method: str = "threshold"):
        self.threshold, self.k_keep, self.method = threshold, k_keep, method

    def optimize(self, layer, tokens, topk_ids, topk_weights, cluster_status=None):
        w = topk_weights
        if self.method == "topk" and self.k_keep > 0:
            kth = w.topk(min(self.k_keep, w.shape[1]), dim=1).values[:, -1:]
            keep = w >= kth
        else:
            keep = w >= self.threshold * w.max(dim=1, keepdim=True).values
        w2 = torch.where(keep, w, torch.zeros_like(w))
        w2 = w2 / w2.sum(dim=1, keepdim=True).clamp_min(1e-20) * w.sum(dim=1, keepdim=True)
        ids2 = torch.where(keep, topk_ids, torch.full_like(topk_ids, -1))
        return tokens, ids2, w2


class TokenBalance(Optimizer):
    """Caps the tokens any expert takes in one step; the overflow (lowest weights first) is dropped."""

    def __init__(self, num_experts: int, capacity_factor: float = 2.0):
        self.E, self.cf = num_experts, capacity_factor

    def optimize(self, layer, tokens, topk_ids, topk_weights, cluster_status=None):
        T, k = topk_ids.shape
        cap = max(1, int(self.cf * T * k / self.E))
        flat_ids, flat_w = topk_ids.reshape(-1), topk_weights.reshape(-1)
        order = torch.argsort(flat_w, descending=True)
        keep = torch.zeros_like(flat_ids, dtype=torch.bool)
        counts = torch.zeros(self.E, dtype=torch.long, device=topk_ids.device)
        for i in order.tolist():
            e = int(flat_ids[i])
            if e >= 0 and counts[e] < cap:
                counts[e] += 1
                keep[i] = True
        ids2 = torch.where(keep, flat_ids, torch.full_like(flat_ids, -1)).view(T, k)
        return tokens, ids2, torch.where(keep.view(T, k), topk_weights, torch.zeros_like(topk_weights))


class ExpertsBalanceOptimizer(Optimizer):
    """Redundant-expert spreading: a token whose expert has several replicas picks the replica by token index."""

    def __init__(self, mapping):
        self.mapping = mapping

    def optimize(self, layer, tokens, topk_ids, topk_weights, cluster_status=None):
        T, k = topk_ids.shape
        place = torch.from_numpy(self.mapping.placement()[layer]).to(topk_ids.device)
        out = topk_ids.clone()
        for e in topk_ids.unique().tolist():
            if e < 0:
                continue
            pos = (place == e).nonzero().flatten()
            if len(pos) == 0:
                continue
            mask = topk_ids == e
            idx = torch.arange(T, device=topk_ids.device).unsqueeze(1).expand(T, k)[mask]
            out[mask] = pos[idx % len(pos)].to(out.dtype)
        return tokens, out, topk_weights
