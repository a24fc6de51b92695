"""Process groups of one engine instance on a single NVSwitch domain.

One process per GPU.  World ranks are laid out ``[dp][tp]`` (TP fastest).  Groups:

* ``world``      every rank of the instance (EP group: experts are sharded over the whole instance)
* ``tp``         attention tensor-parallel group (heads sharded); size 1 = data-parallel attention
* ``dp``         ranks holding the same TP shard, one per attention replica
* ``mlp_tp``     sub-group for the dense MLP layers / shared expert (``dense_mlp_tp_size``)
* ``o_proj_tp``  sub-group that shards o_proj while attention itself is data parallel
* ``cpu``        gloo group over the world for host-side agreement (padding, KV block counts)
* ``pp`` / ``ep`` with pipeline parallelism the layout is ``[pp][inner]``: ``pp`` links the ranks that hold the same
                 inner position in every stage, ``ep`` is the stage's own ranks (the experts of a stage's layers are
                 sharded over them); without pipeline parallelism ``ep`` is the whole instance

The reference additionally builds local/cross groups for its multi-node hierarchical pipelines
(omni/adaptors/vllm/distributed/parallel_state.py:349-635).  One NVSwitch domain has uniform bandwidth, so inside
one box the flat groups above are used; an instance that spans several boxes passes ``ranks_per_domain`` (or
``OMNI_RANKS_PER_DOMAIN``) and gets ``local`` / ``cross`` groups plus the two-stage collectives of
``parallel/hierarchical.py`` in ``ParallelState.hier``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class GroupCoordinator:
    """A process group plus the rank list it was built from (mirrors the accessor surface of the
    reference's GroupCoordinator: all_reduce / all_gather / reduce_scatter / all_to_all / swap)."""
    name: str
    ranks: list[int]
    rank_in_group: int
    group: Optional[dist.ProcessGroup] = None

    @property
    def world_size(self) -> int:
        return len(self.ranks)

    # -- collectives (NCCL or gloo depending on the group backend)
    def all_reduce(self, x: torch.Tensor, op=dist.ReduceOp.SUM, async_op: bool = False):
        if self.world_size == 1:
            return x if not async_op else (x, None)
        work = dist.all_reduce(x, op=op, group=self.group, async_op=async_op)
        return (x, work) if async_op else x

    def all_gather(self, x: torch.Tensor, dim: int = 0, async_op: bool = False):
        if self.world_size == 1:
            return x if not async_op else (x, None)
        x = x.contiguous()
        out = torch.empty((self.world_size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        work = dist.all_gather_into_tensor(out, x, group=self.group, async_op=async_op)
        if async_op:
            return out, work
        if dim == 0:
            return out
        return torch.cat(list(out.view(self.world_size, *x.shape).unbind(0)), dim=dim)

    def reduce_scatter(self, x: torch.Tensor, async_op: bool = False):
        """Sum over the group, scatter along dim 0 (rows must be divisible by the group size)."""
        if self.world_size == 1:
            return x if not async_op else (x, None)
        x = x.contiguous()
        n = x.shape[0] // self.world_size
        if not x.is_cuda:       # gloo has no reduce-scatter: all-reduce and keep this rank's rows
            y = x.clone()
            dist.all_reduce(y, group=self.group)
            out = y[self.rank_in_group * n:(self.rank_in_group + 1) * n].contiguous()
            return (out, None) if async_op else out
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        work = dist.reduce_scatter_tensor(out, x, group=self.group, async_op=async_op)
        return (out, work) if async_op else out

    def all_to_all(self, x: torch.Tensor, out_splits=None, in_splits=None):
        if self.world_size == 1:
            return x
        x = x.contiguous()
        n_out = sum(out_splits) if out_splits is not None else x.shape[0]
        out = torch.empty((n_out,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.group)
        return out

    def swap(self, x: torch.Tensor):
        """Two-rank exchange (omni/adaptors/vllm/distributed/parallel_state.py:61)."""
        assert self.world_size == 2
        peer = self.ranks[1 - self.rank_in_group]
        out = torch.empty_like(x)
        ops = [dist.P2POp(dist.isend, x.contiguous(), peer, self.group), dist.P2POp(dist.irecv, out, peer, self.group)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        return out

    def broadcast(self, x: torch.Tensor, src_in_group: int = 0):
        if self.world_size > 1:
            dist.broadcast(x, src=self.ranks[src_in_group], group=self.group)
        return x

    def barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.group)


@dataclass
class ParallelState:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    tp_size: int = 1
    pp_size: int = 1
    backend: str = "none"
    groups: dict = field(default_factory=dict)
    tp_fused: object = None     # TpFusedContext / TpNcclBaseline when attention runs tensor parallel
    step_max_tokens: int = 0    # largest token-row count of any rank in the current step (0 = not agreed)
    hier: object = None         # HierarchicalGroups when the instance spans more than one NVSwitch domain

    @property
    def dp_size(self) -> int:
        return self.world_size // self.tp_size

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def dp_rank(self) -> int:
        return self.rank // self.tp_size

    @property
    def pp_rank(self) -> int:
        return self.rank // (self.world_size // self.pp_size)

    @property
    def ep_size(self) -> int:
        return self.world_size // self.pp_size

    @property
    def ep_rank(self) -> int:
        return self.rank % self.ep_size

    def group(self, name: str) -> GroupCoordinator:
        return self.groups[name]


_STATE = ParallelState(groups={k: GroupCoordinator(k, [0], 0) for k in ("world", "tp", "dp", "mlp_tp", "o_proj_tp", "cpu", "pp", "ep")})


def get_parallel_state() -> ParallelState:
    return _STATE


def _build(name, all_rank_lists, rank, backend=None) -> GroupCoordinator:
    mine = None
    for ranks in all_rank_lists:
        g = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
        if rank in ranks:
            mine = GroupCoordinator(name, list(ranks), ranks.index(rank), g)
    assert mine is not None
    return mine


def init_distributed(backend: Optional[str] = None, tp_size: int = 1, dense_mlp_tp_size: int = 1,
                     o_proj_tp_size: int = 1, timeout_s: float = 600.0, pp_size: int = 1,
                     ranks_per_domain: int = 0) -> ParallelState:
    """Join the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT and build
    every group.  ``backend`` defaults to nccl with CUDA, gloo otherwise."""
    import datetime

    global _STATE
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank),
                                    timeout=datetime.timedelta(seconds=timeout_s))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s))
    elif torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    assert world % tp_size == 0
    assert world % pp_size == 0
    st = ParallelState(rank=rank, world_size=world, local_rank=local_rank, tp_size=tp_size, pp_size=pp_size, backend=backend)
    if world == 1:
        st.groups = {k: GroupCoordinator(k, [0], 0) for k in ("world", "tp", "dp", "mlp_tp", "o_proj_tp", "cpu", "pp", "ep")}
        _STATE = st
        return st
    allr = list(range(world))
    st.groups["world"] = _build("world", [allr], rank)
    st.groups["tp"] = _build("tp", [allr[i:i + tp_size] for i in range(0, world, tp_size)], rank)
    st.groups["dp"] = _build("dp", [allr[i::tp_size] for i in range(tp_size)], rank)
    m = max(1, min(dense_mlp_tp_size, world))
    st.groups["mlp_tp"] = _build("mlp_tp", [allr[i:i + m] for i in range(0, world, m)], rank)
    o = max(1, min(o_proj_tp_size, world))
    st.groups["o_proj_tp"] = _build("o_proj_tp", [allr[i:i + o] for i in range(0, world, o)], rank)
    st.groups["cpu"] = _build("cpu", [allr], rank, backend="gloo")
    inner = world // pp_size
    st.groups["pp"] = _build("pp", [allr[i::inner] for i in range(inner)], rank)
    st.groups["ep"] = _build("ep", [allr[s * inner:(s + 1) * inner] for s in range(pp_size)], rank)
    rpd = int(ranks_per_domain or os.environ.get("OMNI_RANKS_PER_DOMAIN", "0") or 0)
    if 0 < rpd < world:
        from .hierarchical import build_hierarchical_groups
        st.hier = build_hierarchical_groups(world, rank, rpd)
        st.groups["local"], st.groups["cross"] = st.hier.local, st.hier.cross
    _STATE = st
    return st


def destroy_distributed() -> None:
    global _STATE
    if dist.is_initialized():
        dist.destroy_process_group()
    _STATE = ParallelState(groups={k: GroupCoordinator(k, [0], 0)
                                   for k in ("world", "tp", "dp", "mlp_tp", "o_proj_tp", "cpu", "pp", "ep")})


# -- free-function aliases with the reference's names (omni/adaptors/vllm/distributed/communication_op.py)
def tensor_model_parallel_all_reduce(x):
    return _STATE.group("tp").all_reduce(x)


def tensor_model_parallel_all_gather(x, dim=0):
    return _STATE.group("tp").all_gather(x, dim)


def tensor_model_parallel_reduce_scatter(x):
    return _STATE.group("tp").reduce_scatter(x)


def mlp_all_gather(x, dim=0):
    return _STATE.group("mlp_tp").all_gather(x, dim)


def mlp_reduce_scatter(x):
    return _STATE.group("mlp_tp").reduce_scatter(x)


def all_to_all_world(x, out_splits=None, in_splits=None):
    return _STATE.group("world").all_to_all(x, out_splits, in_splits)
