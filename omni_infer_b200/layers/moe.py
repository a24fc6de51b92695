"""Mixture-of-experts layer: fp32 gate, (grouped) top-k routing with logical->physical remap,
expert-parallel dispatch, grouped expert GEMMs with fused SwiGLU(+quant), combine, shared experts.

Mirrors DeepseekMoE / FusedMoE of the reference (omni/models/common/layers/moe/deepseek_moe.py:121-541,
omni/models/common/layers/moe/fused_moe/layer.py:169-365).  Expert-parallel data paths:

* ``ep_size == 1``  local permutation (csrc/kernels/moe_route.cu)
* ``nccl``          all-to-all over NCCL: the unfused baseline
* ``fused``         one dispatch kernel (quantise + NVLink peer stores + counts) and a combine whose reduce
                    reads peer memory (csrc/kernels/ep_dispatch_combine.cu)

Dedicated shared-expert ranks (``cfg.shared_expert_ranks = R``, the reference's ``redundancy_shared_expert_num``,
omni/models/common/layers/moe/deepseek_moe.py:135-215, 573-600): the first R ranks of the expert-parallel group hold
no routed experts, only the shared expert; the routed experts are spread over the other ranks.  The shared expert is
cut along its intermediate dimension into ``n_shared_experts`` pieces of a routed expert's shape (a SwiGLU MLP is a sum
over such pieces), each piece is an always-selected extra expert with weight 1, and every token sends its row to one of
the R replicas in turn - so the shared expert travels the same dispatch / grouped GEMM / combine path as the routed
ones, and no rank spends time on it beside its routed experts.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..ops import FP8
from ..parallel import get_parallel_state
from .common import Linear, SwiGLUMLP


import os as _os

MULTI_STREAM = _os.environ.get("OMNI_MOE_MULTI_STREAM", "1") == "1"
_SIDE_STREAMS: dict = {}


def _side_stream(device):
    key = (device.type, device.index)
    st = _SIDE_STREAMS.get(key)
    if st is None:
        st = _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return st


class MoEGate(nn.Module):
    def __init__(self, cfg, dtype, device=None):
        super().__init__()
        self.cfg = cfg
        E = cfg.n_routed_experts
        # gate weights stay in the activation dtype; logits come out of the GEMM in fp32
        self.weight = nn.Parameter(torch.empty(E, cfg.hidden_size, dtype=dtype, device=device), requires_grad=False)
        self.e_score_correction_bias = (
            nn.Parameter(torch.zeros(E, dtype=torch.float32, device=device), requires_grad=False)
            if cfg.topk_method == "noaux_tc" else None)

    def logits(self, x):
        return ops.gemm(x, self.weight, out_dtype=torch.float32)


def zipf_router_bias(num_experts: int, layer: int, s: float = 1.2, strength: float = 6.0, seed: int = 0) -> torch.Tensor:
    """Log-popularity bias: the expert of Zipf rank r gets strength * log(p_r / p_max) / log(E), p_r ~ r^-s, with the
    ranks permuted per layer."""
    import math
    g = torch.Generator().manual_seed(seed * 1000 + layer)
    perm = torch.randperm(num_experts, generator=g)
    p = torch.arange(1, num_experts + 1, dtype=torch.float32) ** (-s)
    b = torch.empty(num_experts)
    b[perm] = strength * torch.log(p / p.max()) / math.log(num_experts)
    return b


class MoELayer(nn.Module):
    def __init__(self, cfg, layer_idx: int, *, dtype, device=None, planner=None, ep_backend: str = "auto"):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.moe_index = layer_idx - cfg.first_k_dense_replace
        ps = get_parallel_state()
        self.ep_size, self.ep_rank = ps.ep_size, ps.ep_rank
        self.planner = planner
        E = cfg.n_routed_experts
        redundant = planner.num_redundant_per_rank if planner is not None else 0
        R = int(getattr(cfg, "shared_expert_ranks", 0) or 0) if (self.ep_size > 1 and cfg.n_shared_experts > 0) else 0
        if R:
            if planner is not None:
                raise ValueError("dedicated shared-expert ranks and the expert placement planner cannot be combined")
            if not 0 < R < self.ep_size or E % (self.ep_size - R):
                raise ValueError(f"{R} shared-expert ranks: the {E} routed experts must divide over the other "
                                 f"{self.ep_size - R} ranks")
        self.shared_ranks = R
        self.shared_pieces = cfg.n_shared_experts if R else 0
        assert E % (self.ep_size - R) == 0
        self.slots_per_rank = max(E // (self.ep_size - R) + redundant, self.shared_pieces)
        self.num_physical = self.slots_per_rank * self.ep_size
        self.e_lo = self.ep_rank * self.slots_per_rank          # first physical slot of this rank
        quant = cfg.quantization if cfg.quantization == "fp8_block" else "none"
        self.quant = quant
        H, I = cfg.hidden_size, cfg.moe_intermediate_size
        self.gate = MoEGate(cfg, dtype, device)
        wdt = FP8 if quant == "fp8_block" else dtype
        S = self.slots_per_rank
        # zero-filled, not left as allocated: a redundant slot that no expert has been copied into yet must not hold
        # bit patterns that read as NaN should a stale selector ever point at it
        self.w13 = nn.Parameter(torch.zeros(S, 2 * I, H, dtype=torch.uint8 if wdt == FP8 else wdt, device=device).view(wdt),
                                requires_grad=False)
        self.w2 = nn.Parameter(torch.zeros(S, H, I, dtype=torch.uint8 if wdt == FP8 else wdt, device=device).view(wdt),
                               requires_grad=False)
        if quant == "fp8_block":
            self.w13_scale = nn.Parameter(torch.ones(S, 2 * I // 128, H // 128, dtype=torch.float32, device=device),
                                          requires_grad=False)
            self.w2_scale = nn.Parameter(torch.ones(S, H // 128, (I + 127) // 128, dtype=torch.float32, device=device),
                                         requires_grad=False)
        else:
            self.w13_scale = self.w2_scale = None
        self.shared_experts = None
        if cfg.n_shared_experts > 0 and not R:
            if getattr(cfg, "dense_mlp_tp_size", 1) > 1 and getattr(cfg, "attn_tp_size", 1) == 1:
                # sharded over the mlp_tp sub-group like the dense layers (omni/models/deepseek/deepseek_v3.py:86-136)
                from .linear import ParallelSwiGLUMLP
                self.shared_experts = ParallelSwiGLUMLP(H, I * cfg.n_shared_experts, dtype=dtype, quant=quant, device=device)
            else:
                self.shared_experts = SwiGLUMLP(H, I * cfg.n_shared_experts, dtype=dtype, quant=quant, device=device)
        self.ep_backend = ep_backend
        self.ep_ctx = None          # set by the model runner when the fused NVLink path is enabled
        self.forced_balance = False
        # benchmark aid: fixed per-layer logit bias (load-skew stress); set at construction so that captured decode graphs
        # contain the addition
        self.routing_bias_override = None
        if getattr(cfg, "router_skew", None):
            self.routing_bias_override = zipf_router_bias(cfg.n_routed_experts, self.moe_index, **cfg.router_skew)
            if device is not None:
                self.routing_bias_override = self.routing_bias_override.to(device)

    # ------------------------------------------------------------------ what the local slots hold (no planner)
    def logical_of_slot(self, slot: int):
        """Logical routed expert in local slot ``slot``; ``("shared", j)`` for piece j of the shared expert on a
        shared-expert rank; None for a slot that holds nothing."""
        R = self.shared_ranks
        if R and self.ep_rank < R:
            return ("shared", slot) if slot < self.shared_pieces else None
        per = self.cfg.n_routed_experts // (self.ep_size - R)
        return (self.ep_rank - R) * per + slot if slot < per else None

    def local_slots_of(self, expert: int) -> list:
        """Local slots that hold logical routed expert ``expert`` (none on a shared-expert rank)."""
        R = self.shared_ranks
        if R and self.ep_rank < R:
            return []
        per = self.cfg.n_routed_experts // (self.ep_size - R)
        lo = (self.ep_rank - R) * per
        return [expert - lo] if lo <= expert < lo + per else []

    def _append_shared(self, ids, w):
        """Physical ids of the routed picks (the routed ranks come after the shared ones) plus one always-selected
        column per shared piece, on the replica chosen by (row + this rank) mod R.  Padding rows (id -1) stay out."""
        R, S, ns = self.shared_ranks, self.slots_per_rank, self.shared_pieces
        T = ids.shape[0]
        valid = ids[:, :1] >= 0
        routed = torch.where(ids >= 0, ids + R * S, ids)
        replica = (torch.arange(T, device=ids.device, dtype=ids.dtype) + self.ep_rank) % R
        piece = torch.arange(ns, device=ids.device, dtype=ids.dtype)
        sh = torch.where(valid, replica.view(T, 1) * S + piece.view(1, ns), torch.full((1, 1), -1, dtype=ids.dtype, device=ids.device))
        return torch.cat([routed, sh], 1).contiguous(), torch.cat([w, torch.ones(T, ns, dtype=w.dtype, device=w.device)], 1).contiguous()

    # ------------------------------------------------------------------ routing
    def route(self, x, num_valid=None):
        cfg = self.cfg
        logits = self.gate.logits(x)
        if self.routing_bias_override is not None:
            logits = logits + self.routing_bias_override
        selector = counts = None
        if self.planner is not None:
            selector = self.planner.selector(self.moe_index)
            counts = self.planner.activation_counts(self.moe_index)
        if cfg.topk_method == "noaux_tc":
            kw = dict(mode="sigmoid", bias=self.gate.e_score_correction_bias, n_group=cfg.n_group,
                      topk_group=cfg.topk_group, group_mode="top2sum", renorm=cfg.norm_topk_prob,
                      scale=cfg.routed_scaling_factor)
        elif cfg.topk_method == "group_limited_greedy":
            kw = dict(mode=cfg.scoring_func, n_group=cfg.n_group, topk_group=cfg.topk_group, group_mode="max",
                      renorm=cfg.norm_topk_prob, scale=cfg.routed_scaling_factor)
        else:
            kw = dict(mode=cfg.scoring_func, renorm=cfg.norm_topk_prob, scale=cfg.routed_scaling_factor)
        return ops.router_topk(logits, cfg.num_experts_per_tok, selector=selector, counts=counts,
                               forced_balance=self.forced_balance, num_valid=num_valid, **kw)

    # ------------------------------------------------------------------ expert compute on sorted rows
    def experts(self, xs, x_scale, seg_start, seg_len, row_w, t_hint):
        if self.quant == "fp8_block":
            aq, ascale = ops.gemm(xs, self.w13, w_scale=self.w13_scale, x_scale=x_scale, seg_start=seg_start,
                                  seg_len=seg_len, epi="swiglu_quant", t_hint=t_hint)
            return ops.gemm(aq, self.w2, w_scale=self.w2_scale, x_scale=ascale, seg_start=seg_start, seg_len=seg_len,
                            row_scale=row_w, t_hint=t_hint)
        act = ops.gemm(xs, self.w13, seg_start=seg_start, seg_len=seg_len, epi="swiglu", t_hint=t_hint)
        return ops.gemm(act, self.w2, seg_start=seg_start, seg_len=seg_len, row_scale=row_w, t_hint=t_hint)

    def _shared_on_side_stream(self, x, xq):
        """The shared experts only depend on the layer input, so they run on a second stream beside the router,
        the permutation and the dispatch (small kernels that leave most SMs idle); the routed path joins before it
        adds their output.  Under CUDA-graph capture this becomes a parallel branch of the graph
        (the reference overlaps the same work with its multi-stream option, omni/models/deepseek/deepseek_moe.py)."""
        main = torch.cuda.current_stream()
        side = _side_stream(x.device)
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        with torch.cuda.stream(side):
            shared = self.shared_experts(x, xq=xq)
            done = torch.cuda.Event()
            done.record(side)
        shared.record_stream(main)
        self._shared_done = done
        return shared

    def join_shared(self):
        """Make the current stream wait for the shared-expert branch (no-op when it ran inline)."""
        ev = getattr(self, "_shared_done", None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self._shared_done = None

    def forward(self, x, xq=None, num_valid=None):
        T = x.shape[0]
        k = self.cfg.num_experts_per_tok
        shared = None
        if self.shared_experts is not None:
            if x.is_cuda and MULTI_STREAM:
                shared = self._shared_on_side_stream(x, xq)
            else:
                shared = self.shared_experts(x, xq=xq)
        ids, w = self.route(x, num_valid)
        if self.shared_ranks:
            ids, w = self._append_shared(ids, w)
        if self.ep_size == 1:
            perm = ops.moe_permute(x, ids, w, self.e_lo, self.slots_per_rank, quant=self.quant == "fp8_block", xq_in=xq)
            t_hint = max(16, (T * k + self.slots_per_rank - 1) // self.slots_per_rank)
            y = self.experts(perm.x, perm.x_scale, perm.seg_start, perm.seg_len, perm.row_w, t_hint)
            self.join_shared()
            return ops.moe_combine(y, perm.row_of, T, k, shared=shared)
        if self.ep_ctx is not None and x.is_cuda and x.dtype == torch.bfloat16:
            return self.ep_ctx.moe_forward(self, x, ids, w, shared, xq=xq)
        from ..parallel.ep_nccl import moe_forward_nccl
        return moe_forward_nccl(self, x, ids, w, shared)
