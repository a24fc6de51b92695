"""Two-level collectives for an instance that spans more than one NVSwitch domain.

Inside one domain (one HGX box) every GPU reaches every peer at full NVLink bandwidth and the flat collectives of
``parallel_state`` are the right ones.  An instance spread over several boxes has a fast level (NVLink inside a box)
and a slow one (the network between boxes); sending each byte over the slow level at most once is what the
reference's local / cross group pipelines do for its multi-node deployments
(omni/adaptors/vllm/distributed/parallel_state.py:349-470 build the groups,
omni/adaptors/vllm/distributed/communication_op.py:22-147 are the two-stage and the half-split pipelined forms).

World ranks are laid out ``[domain][local]``: rank ``r`` sits in domain ``r // L`` at local index ``r % L`` with
``L = ranks_per_domain``.  Two groups per rank:

* ``local``  the ``L`` ranks of this rank's domain
* ``cross``  the ranks that share this rank's local index, one per domain

Every function returns exactly what the flat collective over the whole world returns (same row order), so a caller
switches between them by configuration only.  The stage order is chosen so that the slow level carries the small
message: an all-gather crosses domains first (one shard per peer) and fans out inside the domain afterwards; a
reduce-scatter reduces inside the domain first and sends the already reduced block across.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .parallel_state import GroupCoordinator, _build


@dataclass
class HierarchicalGroups:
    ranks_per_domain: int
    num_domains: int
    local: GroupCoordinator
    cross: GroupCoordinator

    @property
    def world_size(self) -> int:
        return self.ranks_per_domain * self.num_domains

    @property
    def domain(self) -> int:
        return self.cross.rank_in_group

    @property
    def local_index(self) -> int:
        return self.local.rank_in_group


def build_hierarchical_groups(world_size: int, rank: int, ranks_per_domain: int,
                              backend: Optional[str] = None) -> HierarchicalGroups:
    """Create the local and cross groups.  Collective over the world: every rank calls it with the same arguments."""
    L = int(ranks_per_domain)
    if L <= 0 or world_size % L:
        raise ValueError(f"ranks_per_domain={L} does not divide the world size {world_size}")
    H = world_size // L
    local = _build("local", [list(range(h * L, (h + 1) * L)) for h in range(H)], rank, backend=backend)
    cross = _build("cross", [list(range(l, world_size, L)) for l in range(L)], rank, backend=backend)
    return HierarchicalGroups(L, H, local, cross)


# ---------------------------------------------------------------------------------------------------------------
# two-stage forms
# ---------------------------------------------------------------------------------------------------------------
def all_gather_two_stage(x: torch.Tensor, hg: HierarchicalGroups, dim: int = 0) -> torch.Tensor:
    """All-gather over the world: across domains first, inside the domain second.  Equal to the flat all-gather
    (blocks in world-rank order along ``dim``)."""
    H, L = hg.num_domains, hg.ranks_per_domain
    x = x.contiguous()
    s1 = hg.cross.all_gather(x, 0)                      # [H * n, ...]   blocks by domain, this local index
    s2 = hg.local.all_gather(s1, 0)                     # [L * H * n, ...]
    out = s2.view(L, H, *x.shape).transpose(0, 1)       # -> [H, L, n, ...] = world-rank order
    if dim == 0:
        return out.reshape(H * L * x.shape[0], *x.shape[1:])
    return torch.cat(list(out.reshape(H * L, *x.shape).unbind(0)), dim=dim)


def reduce_scatter_two_stage(x: torch.Tensor, hg: HierarchicalGroups) -> torch.Tensor:
    """Sum over the world, rank ``r`` keeps row block ``r``: reduce inside the domain first (each local index ends up
    with the partial sums of the ``H`` blocks that its cross group owns), then across domains."""
    H, L = hg.num_domains, hg.ranks_per_domain
    W = H * L
    assert x.shape[0] % W == 0, "rows must divide by the world size"
    n = x.shape[0] // W
    rest = tuple(x.shape[1:])
    # rows are [H, L, n]; the local stage scatters over L, so bring L to the front
    xs = x.view(H, L, n, *rest).transpose(0, 1).reshape(L * H * n, *rest)
    s1 = hg.local.reduce_scatter(xs)                    # [H * n, ...]  partial over this domain
    return hg.cross.reduce_scatter(s1)                  # [n, ...]


def all_reduce_two_stage(x: torch.Tensor, hg: HierarchicalGroups) -> torch.Tensor:
    """Sum over the world with one 1/L-sized message per rank on the slow level: reduce-scatter inside the domain,
    all-reduce of the shard across domains, all-gather inside the domain.  Falls back to local all-reduce followed by
    cross all-reduce when the element count does not divide by ``L``."""
    L = hg.ranks_per_domain
    flat = x.contiguous().view(-1)
    if flat.numel() % L:
        y = hg.local.all_reduce(flat.clone())
        return hg.cross.all_reduce(y).view_as(x)
    shard = hg.local.reduce_scatter(flat)
    shard = hg.cross.all_reduce(shard)
    return hg.local.all_gather(shard, 0).view_as(x)


def all_to_all_two_stage(x: torch.Tensor, hg: HierarchicalGroups) -> torch.Tensor:
    """Equal-split all-to-all over the world (row block ``d`` of the input goes to rank ``d``; row block ``s`` of the
    result came from rank ``s``).  Each block crosses the slow level once, to the peer with the sender's local index
    in the destination domain, and is delivered inside that domain in a second exchange (the rail-aligned routing of
    multi-node expert parallelism; omni/adaptors/vllm/distributed/communication_op.py:269 is the local stage)."""
    H, L = hg.num_domains, hg.ranks_per_domain
    W = H * L
    assert x.shape[0] % W == 0, "rows must divide by the world size"
    n = x.shape[0] // W
    rest = tuple(x.shape[1:])
    s1 = hg.cross.all_to_all(x.contiguous())            # [H_src, L_dst, n]: everything for this domain from (h_src, l)
    s1 = s1.view(H, L, n, *rest).transpose(0, 1).reshape(L * H * n, *rest)   # [L_dst, H_src, n]
    s2 = hg.local.all_to_all(s1)                        # [L_src, H_src, n]
    return s2.view(L, H, n, *rest).transpose(0, 1).reshape(W * n, *rest)     # [H_src, L_src, n] = world order


# ---------------------------------------------------------------------------------------------------------------
# pipelined forms: the tensor is cut into chunks and the slow stage of one chunk runs under the fast stage of the next
# ---------------------------------------------------------------------------------------------------------------
def _wait(work) -> None:
    if work is not None:
        work.wait()


def all_gather_pipelined(x: torch.Tensor, hg: HierarchicalGroups, chunks: int = 2) -> torch.Tensor:
    """``all_gather_two_stage`` along dim 0 with the columns cut in ``chunks`` pieces: the cross stage of piece
    ``i + 1`` is in flight while the local stage of piece ``i`` runs (the reference's half-split two-node pipeline,
    omni/adaptors/vllm/distributed/communication_op.py:94-147, generalised to any chunk count)."""
    H, L = hg.num_domains, hg.ranks_per_domain
    x2 = x.contiguous().view(x.shape[0], -1)
    cols = x2.shape[1]
    chunks = max(1, min(chunks, cols))
    pieces = [p.contiguous() for p in torch.tensor_split(x2, chunks, dim=1)]
    cross = [hg.cross.all_gather(pieces[0], 0, async_op=True)]
    local = []
    for i in range(chunks):
        if i + 1 < chunks:
            cross.append(hg.cross.all_gather(pieces[i + 1], 0, async_op=True))
        s1, w = cross[i]
        _wait(w)
        local.append(hg.local.all_gather(s1, 0, async_op=True))
    outs = []
    for i, (s2, w) in enumerate(local):
        _wait(w)
        n, c = pieces[i].shape
        outs.append(s2.view(L, H, n, c).transpose(0, 1).reshape(H * L * n, c))
    return torch.cat(outs, dim=1).view(H * L * x.shape[0], *x.shape[1:])


def reduce_scatter_pipelined(x: torch.Tensor, hg: HierarchicalGroups, chunks: int = 2) -> torch.Tensor:
    """``reduce_scatter_two_stage`` with the columns cut in ``chunks`` pieces: the local stage of piece ``i + 1`` is
    in flight while the cross stage of piece ``i`` runs (the prefill reduce-scatter pipeline of the reference,
    omni/adaptors/vllm/distributed/communication_op.py:149)."""
    H, L = hg.num_domains, hg.ranks_per_domain
    W = H * L
    assert x.shape[0] % W == 0, "rows must divide by the world size"
    n = x.shape[0] // W
    x2 = x.contiguous().view(x.shape[0], -1)
    cols = x2.shape[1]
    chunks = max(1, min(chunks, cols))
    pieces = []
    for p in torch.tensor_split(x2, chunks, dim=1):
        c = p.shape[1]
        pieces.append(p.reshape(H, L, n, c).transpose(0, 1).reshape(L * H * n, c))
    local = [hg.local.reduce_scatter(pieces[0], async_op=True)]
    cross = []
    for i in range(chunks):
        if i + 1 < chunks:
            local.append(hg.local.reduce_scatter(pieces[i + 1], async_op=True))
        s1, w = local[i]
        _wait(w)
        cross.append(hg.cross.reduce_scatter(s1, async_op=True))
    outs = []
    for s2, w in cross:
        _wait(w)
        outs.append(s2)
    return torch.cat(outs, dim=1).view(n, *x.shape[1:])


def all_gather_round_pipelined(x: torch.Tensor, hg: HierarchicalGroups) -> torch.Tensor:
    """All-gather over the world for a power-of-two number of domains (2, 4, 8 hosts) as rounds of pairwise exchanges:
    in round ``k`` every rank swaps its own shard with the rank of the same local index in domain ``d xor k``, and the
    fan-out of what arrived inside the domain (a local all-gather) is started at once, so it runs while the next
    round's exchange is on the wire.  Every link between two domains carries exactly one shard per rank and round, no
    rank ever waits on a collective that spans all domains (the reference's three-round pairwise pipelines for four
    nodes, omni/adaptors/vllm/distributed/communication_op.py:173-266).  Result: blocks in world-rank order, dim 0."""
    H, L = hg.num_domains, hg.ranks_per_domain
    if H & (H - 1):
        raise ValueError("the pairwise rounds need a power-of-two number of domains")
    x = x.contiguous()
    d = hg.domain
    got = {d: hg.local.all_gather(x, 0, async_op=True)}            # own domain's rows: fan-out starts first
    for k in range(1, H):
        peer = d ^ k
        recv = torch.empty_like(x)
        if hg.cross.world_size > 1:
            ops = [dist.P2POp(dist.isend, x, hg.cross.ranks[peer], hg.cross.group),
                   dist.P2POp(dist.irecv, recv, hg.cross.ranks[peer], hg.cross.group)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        got[peer] = hg.local.all_gather(recv, 0, async_op=True)    # overlaps the next round's exchange
    parts = []
    for h in range(H):
        out, work = got[h]
        _wait(work)
        parts.append(out)                                           # [L * n, ...]: domain h's ranks in local order
    return torch.cat(parts, 0)


# ---------------------------------------------------------------------------------------------------------------
# free functions over the process-wide state (the names the reference's model code calls); flat when the instance
# sits in one domain
# ---------------------------------------------------------------------------------------------------------------
def _state():
    from .parallel_state import get_parallel_state
    return get_parallel_state()


def world_all_gather(x: torch.Tensor, dim: int = 0, pipelined_chunks: int = 0) -> torch.Tensor:
    st = _state()
    if st.hier is None:
        return st.group("world").all_gather(x, dim)
    if pipelined_chunks > 1 and dim == 0:
        return all_gather_pipelined(x, st.hier, pipelined_chunks)
    return all_gather_two_stage(x, st.hier, dim)


def world_reduce_scatter(x: torch.Tensor, pipelined_chunks: int = 0) -> torch.Tensor:
    st = _state()
    if st.hier is None:
        return st.group("world").reduce_scatter(x)
    if pipelined_chunks > 1:
        return reduce_scatter_pipelined(x, st.hier, pipelined_chunks)
    return reduce_scatter_two_stage(x, st.hier)


def world_all_reduce(x: torch.Tensor) -> torch.Tensor:
    st = _state()
    if st.hier is None:
        return st.group("world").all_reduce(x)
    return all_reduce_two_stage(x, st.hier)


def world_all_to_all(x: torch.Tensor) -> torch.Tensor:
    st = _state()
    if st.hier is None:
        return st.group("world").all_to_all(x)
    return all_to_all_two_stage(x, st.hier)


def all_gather_local(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    st = _state()
    return (st.hier.local if st.hier is not None else st.group("world")).all_gather(x, dim)


def all_gather_cross(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    st = _state()
    return st.hier.cross.all_gather(x, dim) if st.hier is not None else x


def reduce_scatter_local(x: torch.Tensor) -> torch.Tensor:
    st = _state()
    return (st.hier.local if st.hier is not None else st.group("world")).reduce_scatter(x)


def reduce_scatter_cross(x: torch.Tensor) -> torch.Tensor:
    st = _state()
    return st.hier.cross.reduce_scatter(x) if st.hier is not None else x


def all_to_all_local(x: torch.Tensor) -> torch.Tensor:
    st = _state()
    return (st.hier.local if st.hier is not None else st.group("world")).all_to_all(x)
