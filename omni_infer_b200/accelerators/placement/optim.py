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


def _replica_table(mapping, layer: int, device):
    """positions [experts, max_replicas] (-1 padded) and counts [experts] of a layer's replicas, in position order."""
    place = torch.as_tensor(mapping.placement()[layer], device=device)
    experts = int(place.max().item()) + 1 if place.numel() else 0
    experts = max(experts, getattr(mapping, "experts", experts))
    lists = [[] for _ in range(experts)]
    for pos, e in enumerate(place.tolist()):
        if e >= 0:
            lists[e].append(pos)
    width = max(1, max((len(x) for x in lists), default=1))
    table = torch.full((experts, width), -1, dtype=torch.long, device=device)
    for e, x in enumerate(lists):
        if x:
            table[e, :len(x)] = torch.tensor(x, dtype=torch.long, device=device)
    counts = torch.tensor([len(x) for x in lists], dtype=torch.long, device=device).clamp_min(1)
    return table, counts


class HEATExpertsBalancer(Optimizer):
    """Host-aware replica choice (reference: heat_optimizer.py, device-specific mode): a token's expert goes to the
    replica on this rank if there is one, else to one on this host, else to the replica picked by the rank's offset
    (``rank % replicas``, or one global offset for all ranks), so that the ranks spread over the replicas."""

    def __init__(self, mapping, rank: int = 0, ranks_per_host: int = 8, global_offset: bool = False):
        self.mapping, self.rank, self.rph, self.global_offset = mapping, rank, max(1, ranks_per_host), global_offset
        self._tables: dict = {}

    def table(self, layer: int, device) -> torch.Tensor:
        """logical expert -> physical position for this rank."""
        key = (layer, str(device))
        if key not in self._tables:
            pos, cnt = _replica_table(self.mapping, layer, device)
            S = self.mapping.slots_per_rank
            owner = torch.where(pos >= 0, pos // S, torch.full_like(pos, -10 ** 6))
            local = owner == self.rank
            same_host = (owner // self.rph) == (self.rank // self.rph)
            offset = torch.zeros_like(cnt) if self.global_offset else self.rank % cnt
            pick = pos.gather(1, offset.unsqueeze(1)).squeeze(1)
            first = lambda mask: torch.where(mask.any(1), pos.gather(1, mask.float().argmax(1, keepdim=True)).squeeze(1), pick)  # noqa: E731
            pick = first(same_host)
            pick = torch.where(local.any(1), pos.gather(1, local.float().argmax(1, keepdim=True)).squeeze(1), pick)
            self._tables[key] = pick
        return self._tables[key]

    def invalidate(self) -> None:
        self._tables.clear()

    def optimize(self, layer, tokens, topk_ids, topk_weights, cluster_status=None):
        t = self.table(layer, topk_ids.device)
        out = torch.where(topk_ids >= 0, t[topk_ids.clamp_min(0)], topk_ids)
        return tokens, out, topk_weights


class Redundant2ExpertsBalancer(Optimizer):
    """Replica choice by token (reference: redundant_experts_optimizer.py, not device-specific): pair (token i, choice
    j) of expert e goes to replica ``(i + j + rank) % replicas(e)``: even spreading without any state."""

    def __init__(self, mapping, rank: int = 0):
        self.mapping, self.rank = mapping, rank
        self._tables: dict = {}

    def optimize(self, layer, tokens, topk_ids, topk_weights, cluster_status=None):
        key = (layer, str(topk_ids.device))
        if key not in self._tables:
            self._tables[key] = _replica_table(self.mapping, layer, topk_ids.device)
        pos, cnt = self._tables[key]
        T, k = topk_ids.shape
        ids = topk_ids.clamp_min(0)
        turn = (torch.arange(T, device=ids.device).unsqueeze(1) + torch.arange(k, device=ids.device).unsqueeze(0) + self.rank) % cnt[ids]
        out = pos[ids, turn]
        return tokens, torch.where(topk_ids >= 0, out, topk_ids), topk_weights


class ResDisExpertsBalancer(Optimizer):
    """Residual dispatch (reference: resdispatch_optimizer.py): the pairs of one expert are dealt over its replicas
    in proportion to the room each replica's rank has left, ``room = max(target - load, 0)`` with ``cluster_status`` =
    tokens already on every rank (``[world]``) and the mean as target; without loads, or when nobody has room, the deal
    is even (or random with ``random=True``).  ``max_count`` bounds how many pairs of one expert are balanced per step,
    the rest goes to the first replica (the reference's cap on its per-step work)."""

    def __init__(self, mapping, rank: int = 0, random: bool = False, max_count: int = 1 << 30, seed: int = 0):
        self.mapping, self.rank, self.random, self.max_count = mapping, rank, random, max_count
        self._gen = torch.Generator().manual_seed(seed)

    def optimize(self, layer, tokens, topk_ids, topk_weights, cluster_status=None):
        dev = topk_ids.device
        pos, cnt = _replica_table(self.mapping, layer, dev)
        S = self.mapping.slots_per_rank
        out = topk_ids.clone()
        loads = None if cluster_status is None else torch.as_tensor(cluster_status, dtype=torch.float32, device=dev)
        for e in topk_ids.unique().tolist():
            if e < 0 or cnt[e] <= 1:
                if e >= 0:
                    out[topk_ids == e] = pos[e, 0].to(out.dtype)
                continue
            mask = topk_ids == e
            n = int(mask.sum())
            reps = pos[e, :cnt[e]]
            share = torch.full((len(reps),), 1.0 / len(reps))
            if loads is not None:
                room = (loads.mean() - loads[(reps // S).cpu()].cpu()).clamp_min(0)
                if float(room.sum()) > 0:
                    share = room / room.sum()
            m = min(n, self.max_count)
            if self.random:
                pick = torch.multinomial(share, m, replacement=True, generator=self._gen)
            else:
                # largest-remainder apportionment of m pairs, then dealt in replica order
                quota = share * m
                base = quota.floor().long()
                rest = m - int(base.sum())
                if rest > 0:
                    base[torch.argsort(quota - base.float(), descending=True)[:rest]] += 1
                pick = torch.repeat_interleave(torch.arange(len(reps)), base)
            pick = torch.cat([pick, torch.zeros(n - m, dtype=torch.long)]) if n > m else pick
            out[mask] = reps[pick.to(dev)].to(out.dtype)
        return tokens, out, topk_weights


REGISTRY = {"AdaRouter": AdaRouter, "TokenBalance": TokenBalance, "ExpertsBalanceOptimizer": ExpertsBalanceOptimizer,
            "HEAT_ExpertsBalancer": HEATExpertsBalancer, "Redundant2ExpertsBalancer": Redundant2ExpertsBalancer,
            "ResDis_ExpertsBalancer": ResDisExpertsBalancer}


def create_optimizers(config: list, mapping=None, rank: int = 0, num_experts: int = 0) -> list:
    """``Optimizers:`` section of the planner's config -> instances (reference: optimizers_loader.py).  Entries are
    one-key dicts ``{"<module>.<Class>" or "<Class>": {keyword arguments}}``; the module part of the reference's
    names is accepted and ignored."""
    out = []
    for entry in config or []:
        (name, kw), = entry.items()
        cls_name = name.split(".")[-1]
        if cls_name not in REGISTRY:
            raise ValueError(f"unsupported optimizer: {name}")
        cls, kw = REGISTRY[cls_name], dict(kw or {})
        if cls is AdaRouter:
            out.append(cls(**kw))
        elif cls is TokenBalance:
            out.append(cls(kw.pop("num_experts", num_experts), **kw))
        elif cls is ExpertsBalanceOptimizer:
            out.append(cls(mapping))
        else:
            out.append(cls(mapping, rank=rank, **kw))
    return out
