"""Parallel linear layers over the process groups of one instance.

The reference keeps a family of column / row parallel linears whose collectives differ by where the layer sits
(omni/models/common/layers/linear.py:40-1245): merged column-parallel, row-parallel with all-reduce or
reduce-scatter, the DP->TP o_proj whose inputs come from an all-to-all of attention outputs, a column-parallel
linear that gathers quantised activations, replicated merged linears, and the dense MLP that all-gathers token
rows over the ``mlp_tp`` sub-group and reduce-scatters its output (omni/models/deepseek/deepseek_v3.py:86-136).

Here every layer is a :class:`~omni_infer_b200.layers.common.Linear` holding this rank's shard plus a
:class:`GroupCoordinator`; the GEMM is the same sm_100a kernel as everywhere else and the collective is the
group's (NCCL on GPUs, gloo on CPU ranks).  The attention tensor-parallel path has its own GEMMs with the
collective inside (parallel/tp_fused.py); the layers below serve the sub-groups that shard the dense MLP, the
shared expert and o_proj while attention stays data parallel.

Every sharded parameter carries ``tp_slice_fn`` / ``tp_full_shape`` so that checkpoint loading and the seeded
random initialisation cut this rank's slice out of the full tensor: a sharded model is the unsharded model."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..parallel.parallel_state import GroupCoordinator, get_parallel_state
from .common import Linear


def _mark_rows(lin: Linear, full_rows: int, rank: int, world: int, unit_rows: int) -> None:
    """``lin`` holds rows [rank * unit_rows, +unit_rows) of a [full_rows, K] weight."""
    K = lin.in_features
    lin.weight.tp_slice_fn = lambda full: full[rank * unit_rows:(rank + 1) * unit_rows]
    lin.weight.tp_full_shape = (full_rows, K)
    if lin.weight_scale is not None:
        assert unit_rows % 128 == 0, "e4m3 row shards must align to the 128x128 scale blocks"
        lin.weight_scale.tp_slice_fn = lambda full: full[rank * unit_rows // 128:(rank + 1) * unit_rows // 128]


def _mark_cols(lin: Linear, full_cols: int, rank: int, world: int, unit_cols: int) -> None:
    """``lin`` holds columns [rank * unit_cols, +unit_cols) of a [N, full_cols] weight."""
    N = lin.out_features
    lin.weight.tp_slice_fn = lambda full: full[:, rank * unit_cols:(rank + 1) * unit_cols].contiguous()
    lin.weight.tp_full_shape = (N, full_cols)
    if lin.weight_scale is not None:
        assert unit_cols % 128 == 0, "e4m3 column shards must align to the 128x128 scale blocks"
        lin.weight_scale.tp_slice_fn = lambda full: full[:, rank * unit_cols // 128:(rank + 1) * unit_cols // 128].contiguous()


def _pad_rows(x: torch.Tensor, rows: int) -> torch.Tensor:
    if x.shape[0] == rows:
        return x
    return torch.cat([x, x.new_zeros(rows - x.shape[0], *x.shape[1:])], 0)


def group_max_rows(group: GroupCoordinator, rows: int) -> int:
    """Rows every rank of the group pads to.  The model runner publishes the step's maximum over all ranks
    (``ParallelState.step_max_tokens``, agreed on the host group before the forward); without it the layer asks
    the group itself."""
    ps = get_parallel_state()
    m = int(getattr(ps, "step_max_tokens", 0) or 0)
    if m >= rows:
        return m
    if group.world_size == 1:
        return rows
    t = torch.tensor([rows], dtype=torch.int64)
    import torch.distributed as dist
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ps.group("cpu").group)
    return int(t.item())


class MergedColumnParallelLinear(Linear):
    """Several column-parallel projections of the same input stored as one weight: every part is sharded over the
    group on its own, and this rank's shards are stacked (reference: AscendMergedColumnParallelLinear, linear.py:40)."""

    def __init__(self, in_features: int, part_sizes: list, group: GroupCoordinator, *, dtype=torch.bfloat16,
                 quant: str = "none", device=None):
        W, r = group.world_size, group.rank_in_group
        assert all(p % W == 0 for p in part_sizes)
        local = [p // W for p in part_sizes]
        super().__init__(in_features, sum(local), dtype=dtype, quant=quant, device=device)
        self.group, self.part_sizes, self.local_sizes = group, list(part_sizes), local
        full = sum(part_sizes)
        offs = [sum(part_sizes[:i]) for i in range(len(part_sizes))]
        if W > 1:
            def rows(t, unit=1):
                return torch.cat([t[(o + r * l) // unit:(o + (r + 1) * l) // unit] for o, l in zip(offs, local)], 0)
            self.weight.tp_slice_fn = rows
            self.weight.tp_full_shape = (full, in_features)
            if self.weight_scale is not None:
                assert all(l % 128 == 0 for l in local)
                self.weight_scale.tp_slice_fn = lambda t: rows(t, 128)


class RowParallelLinear(Linear):
    """Input features sharded over the group; the partial sums are all-reduced, or reduce-scattered over token rows
    (reference: AscendRowParallelLinear linear.py:238, RowParallelLinearWithReduceScatter linear.py:587)."""

    def __init__(self, in_features: int, out_features: int, group: GroupCoordinator, *, reduce: str = "all_reduce",
                 dtype=torch.bfloat16, quant: str = "none", device=None):
        assert reduce in ("all_reduce", "reduce_scatter", "none")
        W, r = group.world_size, group.rank_in_group
        assert in_features % W == 0
        super().__init__(in_features // W, out_features, dtype=dtype, quant=quant, device=device)
        self.group, self.reduce = group, reduce
        if W > 1:
            _mark_cols(self, in_features, r, W, in_features // W)

    def forward(self, x, xq=None):
        y = Linear.forward(self, x, xq=xq)
        if self.group.world_size == 1 or self.reduce == "none":
            return y
        if self.reduce == "all_reduce":
            return self.group.all_reduce(y)
        return self.group.reduce_scatter(y)


class ColumnParallelLinearQuantGather(Linear):
    """Column-parallel linear whose input rows are sharded over the group: the rows are quantised to e4m3 first and
    gathered in that form (half the bytes on the wire), then multiplied (reference: linear.py:523)."""

    def __init__(self, in_features: int, out_features: int, group: GroupCoordinator, *, dtype=torch.bfloat16,
                 quant: str = "none", device=None):
        W, r = group.world_size, group.rank_in_group
        assert out_features % W == 0
        super().__init__(in_features, out_features // W, dtype=dtype, quant=quant, device=device)
        self.group = group
        if W > 1:
            _mark_rows(self, out_features, r, W, out_features // W)

    def forward(self, x_shard):
        g = self.group
        if self.quant == "fp8_block" and g.world_size > 1:
            q, s = ops.quant_fp8_block(x_shard)                 # s: [K/128, rows]
            rows = x_shard.shape[0]
            qa = g.all_gather(q.view(torch.uint8)).view(q.dtype)
            sa = g.all_gather(s[:, :rows].t().contiguous()).t().contiguous()
            return Linear.forward(self, None, xq=(qa, sa))
        return Linear.forward(self, g.all_gather(x_shard))


class MergedReplicatedLinear(Linear):
    """Several projections of one input as a single replicated weight (reference: linear.py:620)."""

    def __init__(self, in_features: int, part_sizes: list, *, dtype=torch.bfloat16, quant: str = "none", device=None):
        super().__init__(in_features, sum(part_sizes), dtype=dtype, quant=quant, device=device)
        self.part_sizes = list(part_sizes)

    def forward(self, x, xq=None):
        y = Linear.forward(self, x, xq=xq)
        return torch.split(y, self.part_sizes, dim=-1)


class DP2TPRowParallelLinear(Linear):
    """o_proj sharded over the ``o_proj_tp`` group although attention is data parallel
    (reference: DP2TPRowParallelLinear, linear.py:356-520, forward :488-504).

    Every rank arrives with the attention output of its own tokens for all heads, [T, H * vd].  An all-to-all inside
    the group turns that into all the group's tokens for this rank's slice of the heads, [W * T, H * vd / W]; the
    weight holds the matching input columns; the partial sums are reduce-scattered back so that every rank ends
    up with the full projection of its own tokens.  Ranks pad to a common row count first."""

    def __init__(self, in_features: int, out_features: int, group: GroupCoordinator, *, dtype=torch.bfloat16,
                 quant: str = "none", device=None):
        W, r = group.world_size, group.rank_in_group
        assert in_features % W == 0
        super().__init__(in_features // W, out_features, dtype=dtype, quant=quant, device=device)
        self.group = group
        self.full_in_features = in_features
        if W > 1:
            _mark_cols(self, in_features, r, W, in_features // W)

    def forward(self, x, xq=None):
        g = self.group
        W = g.world_size
        if W == 1:
            return Linear.forward(self, x, xq=xq)
        T = x.shape[0]
        Tm = group_max_rows(g, T)
        x = _pad_rows(x, Tm)
        c = self.full_in_features // W
        # [Tm, W, c] -> [W, Tm, c]: block j goes to rank j and holds this rank's tokens for rank j's columns
        send = x.view(Tm, W, c).transpose(0, 1).contiguous().view(W * Tm, c)
        recv = g.all_to_all(send)                               # [W * Tm, c]: block i = rank i's tokens, my columns
        y = Linear.forward(self, recv)                          # partial sums for every token of the group
        return g.reduce_scatter(y)[:T]


class ParallelSwiGLUMLP(nn.Module):
    """Dense MLP (or shared expert) sharded over the ``mlp_tp`` sub-group while attention is data parallel:
    all-gather the token rows of the group, gate/up column-parallel with the SwiGLU in the GEMM epilogue, down
    row-parallel, reduce-scatter back to this rank's rows (reference: ParallelDeepseekMLP,
    omni/models/deepseek/deepseek_v3.py:86-136)."""

    def __init__(self, hidden: int, inter: int, group: Optional[GroupCoordinator] = None, *, dtype=torch.bfloat16,
                 quant: str = "none", device=None):
        super().__init__()
        self.group = group if group is not None else get_parallel_state().group("mlp_tp")
        W = self.group.world_size
        assert inter % W == 0
        self.quant = quant
        self.gate_up_proj = MergedColumnParallelLinear(hidden, [inter, inter], self.group, dtype=dtype, quant=quant, device=device)
        self.down_proj = RowParallelLinear(inter, hidden, self.group, reduce="none", dtype=dtype, quant=quant, device=device)
        self.can_fuse_swiglu = (inter // W) % 128 == 0

    def forward(self, x, xq=None):
        g = self.group
        T = x.shape[0]
        if g.world_size > 1:
            Tm = group_max_rows(g, T)
            x = g.all_gather(_pad_rows(x, Tm))
            xq = None                                  # the quantised form belonged to this rank's rows only
        gu, dn = self.gate_up_proj, self.down_proj
        if self.quant == "fp8_block":
            if xq is None:
                xq = ops.quant_fp8_block(x)
            aq = ops.gemm(xq[0], gu.weight, w_scale=gu.weight_scale, x_scale=xq[1], epi="swiglu_quant")
            y = ops.gemm(aq[0], dn.weight, w_scale=dn.weight_scale, x_scale=aq[1])
        else:
            act = ops.gemm(x, gu.weight, epi="swiglu")
            y = ops.gemm(act, dn.weight)
        if g.world_size > 1:
            y = g.reduce_scatter(y)[:T]
        return y


# ---------------------------------------------------------------------------------------------------------------
# Sequence-sharded ("flash-comm") family: between the blocks every rank keeps only its rows of the hidden states;
# a column-parallel layer gathers the rows on the way in, a row-parallel layer scatters the sums on the way out, so the
# residual stream, the norms and everything else elementwise run on 1/W of the tokens
# (reference: RowParallelFlashCommLinear / ColumnParallelFlashCommLinear / QKVParallelFlashCommLinear /
# MergedColumnParallelFlashCommLinear, omni/models/common/layers/linear.py:955-1245; used by qwen/qwen2.py).
# ---------------------------------------------------------------------------------------------------------------
class RowParallelLinearWithReduceScatter(RowParallelLinear):
    """Row-parallel linear whose partial sums are reduce-scattered over token rows (reference: linear.py:587)."""

    def __init__(self, in_features: int, out_features: int, group: GroupCoordinator, **kw):
        kw.pop("reduce", None)
        super().__init__(in_features, out_features, group, reduce="reduce_scatter", **kw)


class RowParallelLinearCross(RowParallelLinear):
    """Row-parallel linear over the cross group of an instance that spans several NVSwitch domains (one rank per
    domain with the same local index); inside one domain it is the plain layer over the given group
    (reference: RowParallelLinearCross, linear.py:764)."""

    def __init__(self, in_features: int, out_features: int, group: Optional[GroupCoordinator] = None, **kw):
        ps = get_parallel_state()
        if group is None:
            group = ps.group("cross") if getattr(ps, "hier", None) is not None else ps.group("world")
        super().__init__(in_features, out_features, group, **kw)


class ColumnParallelFlashCommLinear(Linear):
    """Output features sharded over the group; the input arrives sharded by token rows and is all-gathered first
    (``gather_input=False`` for an input that is already whole)."""

    def __init__(self, in_features: int, out_features: int, group: GroupCoordinator, *, gather_input: bool = True,
                 bias: bool = False, dtype=torch.bfloat16, quant: str = "none", device=None):
        W, r = group.world_size, group.rank_in_group
        assert out_features % W == 0
        super().__init__(in_features, out_features // W, bias=bias, dtype=dtype, quant=quant, device=device)
        self.group, self.gather_input = group, gather_input
        if W > 1:
            _mark_rows(self, out_features, r, W, out_features // W)
            if self.bias is not None:
                u = out_features // W
                self.bias.tp_slice_fn = lambda full: full[r * u:(r + 1) * u]
                self.bias.tp_full_shape = (out_features,)

    def forward(self, x, xq=None):
        if self.gather_input and self.group.world_size > 1:
            x, xq = self.group.all_gather(x), None
        return Linear.forward(self, x, xq=xq)


class MergedColumnParallelFlashCommLinear(MergedColumnParallelLinear):
    """Merged column-parallel projections (gate / up) of a row-sharded input."""

    def __init__(self, in_features: int, part_sizes: list, group: GroupCoordinator, *, gather_input: bool = True, **kw):
        super().__init__(in_features, part_sizes, group, **kw)
        self.gather_input = gather_input

    def forward(self, x, xq=None):
        if self.gather_input and self.group.world_size > 1:
            x, xq = self.group.all_gather(x), None
        return Linear.forward(self, x, xq=xq)


class RowParallelFlashCommLinear(RowParallelLinear):
    """Input features sharded over the group; the sums go back to row shards (``reduce="reduce_scatter"``, the
    default) or stay whole on every rank (``"all_reduce"``, for the last layer before something that needs all rows)."""

    def __init__(self, in_features: int, out_features: int, group: GroupCoordinator, *, reduce: str = "reduce_scatter", **kw):
        super().__init__(in_features, out_features, group, reduce=reduce, **kw)


class QKVParallelFlashCommLinear(Linear):
    """Merged q / k / v projection with the heads sharded over the group: query heads divide, K/V heads divide when
    there are enough of them and are otherwise held by every rank whose query heads read them; row-sharded input."""

    def __init__(self, hidden: int, head_dim: int, num_heads: int, num_kv_heads: int, group: GroupCoordinator, *,
                 gather_input: bool = True, bias: bool = False, dtype=torch.bfloat16, quant: str = "none", device=None):
        from .gqa import shard_heads
        W, r = group.world_size, group.rank_in_group
        hq, hkv, kv0 = shard_heads(num_heads, num_kv_heads, W, r)
        D = head_dim
        super().__init__(hidden, (hq + 2 * hkv) * D, bias=bias, dtype=dtype, quant=quant, device=device)
        self.group, self.gather_input = group, gather_input
        self.num_heads, self.num_kv_heads, self.head_dim = hq, hkv, D
        if W > 1:
            offs = (0, num_heads * D, (num_heads + num_kv_heads) * D)
            blocks = [(offs[0] + r * hq * D, offs[0] + (r + 1) * hq * D), (offs[1] + kv0 * D, offs[1] + (kv0 + hkv) * D),
                      (offs[2] + kv0 * D, offs[2] + (kv0 + hkv) * D)]
            self.weight.tp_slice_fn = lambda full: torch.cat([full[a:b] for a, b in blocks], 0)
            self.weight.tp_full_shape = ((num_heads + 2 * num_kv_heads) * D, hidden)
            if self.weight_scale is not None:
                assert D % 128 == 0, "e4m3 head shards must align to the 128x128 scale blocks"
                self.weight_scale.tp_slice_fn = lambda full: torch.cat([full[a // 128:b // 128] for a, b in blocks], 0)
            if self.bias is not None:
                self.bias.tp_slice_fn = lambda full: torch.cat([full[a:b] for a, b in blocks], 0)
                self.bias.tp_full_shape = ((num_heads + 2 * num_kv_heads) * D,)

    def forward(self, x, xq=None):
        """Returns (q, k, v) of this rank's heads for all rows."""
        if self.gather_input and self.group.world_size > 1:
            x, xq = self.group.all_gather(x), None
        y = Linear.forward(self, x, xq=xq)
        D = self.head_dim
        return torch.split(y, [self.num_heads * D, self.num_kv_heads * D, self.num_kv_heads * D], dim=-1)
