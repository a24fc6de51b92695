"""Grouped-query attention (Qwen2 / Qwen3-MoE) over a paged K/V cache
(reference backend: omni/models/common/layers/attention/backend/attention.py:507-702).

With ``attn_tp_size`` > 1 the query heads are sharded over the ranks and so are the K/V heads; when there are fewer
K/V heads than ranks each K/V head is held by the ``W / Hkv`` ranks whose query heads use it (the layout of the
reference's QKVParallelLinear users, omni/models/qwen/qwen2.py:100-180).  Every rank then caches only its own K/V
heads, and the hidden states travel sharded by token rows between the attention blocks (``forward_tp``)."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from .common import AttnMetadata, Linear, RMSNorm


class GQAAttention(nn.Module):
    def __init__(self, cfg, layer_idx: int, *, dtype, device=None, cos_sin=None):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.Hq_all, self.Hkv_all, self.D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.tp_world, self.tp_rank = int(getattr(cfg, "attn_tp_size", 1)), int(getattr(cfg, "attn_tp_rank", 0))
        self.Hq, self.Hkv, self.kv_head0 = shard_heads(self.Hq_all, self.Hkv_all, self.tp_world, self.tp_rank)
        quant = cfg.quantization if cfg.quantization == "fp8_block" else "none"
        self.quant = quant
        self.qkv_proj = Linear(cfg.hidden_size, (self.Hq + 2 * self.Hkv) * self.D, dtype=dtype, quant=quant,
                               bias=cfg.attention_bias, device=device)
        self.o_proj = Linear(self.Hq * self.D, cfg.hidden_size, dtype=dtype, quant=quant, device=device)
        self.q_norm = RMSNorm(self.D, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.k_norm = RMSNorm(self.D, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.scale = self.D ** -0.5
        self.cos_sin = cos_sin
        if self.tp_world > 1:
            self._mark_tp_shards()

    def process_weights_after_loading(self):
        pass

    # ------------------------------------------------------------------ tensor-parallel sharding
    def tp_ckpt_rows(self, kind: str):
        """For the checkpoint tensor ``q`` / ``k`` / ``v`` _proj: (rows of that tensor this rank holds, rows of the
        local merged qkv_proj they go to)."""
        D, r = self.D, self.tp_rank
        if kind == "q":
            return (r * self.Hq * D, (r + 1) * self.Hq * D), (0, self.Hq * D)
        src = (self.kv_head0 * D, (self.kv_head0 + self.Hkv) * D)
        d0 = (self.Hq if kind == "k" else self.Hq + self.Hkv) * D
        return src, (d0, d0 + self.Hkv * D)

    def _mark_tp_shards(self):
        """Slices of the whole-model tensors for the loaders that draw or read full tensors: merged qkv rows by head
        (column parallel), o_proj columns by query head (row parallel)."""
        D, Hq_all, Hkv_all = self.D, self.Hq_all, self.Hkv_all
        offs = {"q": 0, "k": Hq_all * D, "v": (Hq_all + Hkv_all) * D}
        blocks = [(offs[k] + self.tp_ckpt_rows(k)[0][0], offs[k] + self.tp_ckpt_rows(k)[0][1]) for k in ("q", "k", "v")]
        fp8 = self.quant == "fp8_block"
        if fp8:
            assert D % 128 == 0, "fp8 shards must be aligned to the 128x128 scale blocks"
        w = self.qkv_proj.weight
        w.tp_slice_fn = lambda full: torch.cat([full[a:b] for a, b in blocks], 0)
        w.tp_full_shape = ((Hq_all + 2 * Hkv_all) * D, self.cfg.hidden_size)
        if fp8:
            self.qkv_proj.weight_scale.tp_slice_fn = lambda full: torch.cat([full[a // 128:b // 128] for a, b in blocks], 0)
        c0, c1 = self.tp_rank * self.Hq * D, (self.tp_rank + 1) * self.Hq * D
        o = self.o_proj.weight
        o.tp_slice_fn = lambda full: full[:, c0:c1].contiguous()
        o.tp_full_shape = (self.cfg.hidden_size, Hq_all * D)
        if fp8:
            self.o_proj.weight_scale.tp_slice_fn = lambda full: full[:, c0 // 128:c1 // 128].contiguous()

    def forward(self, x, md: AttnMetadata, kv_cache, xq=None):
        md = _omni_view(md, self.layer_idx)
        return self.o_proj(self._attend(self.qkv_proj(x, xq=xq), md, kv_cache))

    def forward_tp(self, x_shard, xq_shard, md: AttnMetadata, kv_cache, residual_shard, post_norm, tp):
        """Heads sharded over the ranks, hidden states sharded by token rows outside the attention block: the row
        all-gather runs inside the qkv projection, o_proj inside the reduce-scatter, which also adds the residual and
        applies ``post_norm``.  Returns (new residual rows, normalised rows)."""
        md = _omni_view(md, self.layer_idx)
        Tp = x_shard.shape[0] * tp.world          # padded token rows of the step
        T = md.positions.shape[0]                 # real token rows (<= Tp)
        lin = self.qkv_proj
        if self.quant == "fp8_block":
            qkv, _, _ = tp.allgather_gemm(xq_shard[0], lin.weight, total_rows=Tp, w_scale=lin.weight_scale,
                                          x_scale_shard=xq_shard[1])
        else:
            qkv, _, _ = tp.allgather_gemm(x_shard, lin.weight, total_rows=Tp)
        qkv = qkv[:T]
        if lin.bias is not None:
            qkv = qkv + lin.bias
        o = self._attend(qkv.contiguous(), md, kv_cache)
        if T < Tp:   # padding rows contribute zeros to the sum
            o = torch.cat([o, o.new_zeros(Tp - T, o.shape[1])], 0)
        op = self.o_proj
        if self.quant == "fp8_block":
            oq, os_ = ops.quant_fp8_block(o)
            return tp.gemm_reduce_scatter(oq, op.weight, w_scale=op.weight_scale, x_scale=os_, residual=residual_shard,
                                          norm_weight=post_norm.weight, eps=post_norm.eps)
        return tp.gemm_reduce_scatter(o, op.weight, residual=residual_shard, norm_weight=post_norm.weight, eps=post_norm.eps)

    def _attend(self, qkv, md: AttnMetadata, kv_cache):
        """RoPE (+ q/k norm) and cache write on the merged projection, then attention; returns [T, Hq * D]."""
        T = qkv.shape[0]
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        k_cache, v_cache = kv_cache
        ops.rope_qk_cache(qkv, Hq, Hkv, D, self.cos_sin, md.positions, md.slot_mapping, k_cache, v_cache,
                          self.q_norm.weight if self.q_norm is not None else None,
                          self.k_norm.weight if self.k_norm is not None else None, self.cfg.rms_norm_eps)
        v3 = qkv.view(T, Hq + 2 * Hkv, D)
        q = v3[:, :Hq]
        if md.is_prefill:
            if md.kv_gather_slots is not None:
                k = k_cache.view(-1, Hkv, D)[md.kv_gather_slots]
                v = v_cache.view(-1, Hkv, D)[md.kv_gather_slots]
            else:
                k, v = v3[:, Hq:Hq + Hkv], v3[:, Hq + Hkv:]
            o = ops.attention.gqa_prefill(q, k, v, md.cu_q, md.cu_k, self.scale, md.max_q, md.max_k)
        else:
            o = ops.attention.gqa_decode(q.contiguous(), k_cache, v_cache, md.block_table, md.q_seq_lens, self.scale,
                                         md.max_seq_len)
        return o.reshape(T, Hq * D)


def shard_heads(hq_all: int, hkv_all: int, world: int, rank: int):
    """(query heads, K/V heads, first global K/V head) of one rank.  K/V heads divide over the ranks when there are
    enough of them; otherwise each one is replicated on the ranks whose query heads read it."""
    assert hq_all % world == 0, "query heads must divide over the tensor-parallel ranks"
    assert hkv_all % world == 0 or world % hkv_all == 0, "K/V heads must divide the ranks or be divided by them"
    return hq_all // world, max(1, hkv_all // world), rank * hkv_all // world


def _omni_view(md: AttnMetadata, layer_idx: int) -> AttnMetadata:
    """Metadata as a compressed Omni-Attention layer sees it: its own slot mapping and, for decode, the per-request
    window table and attended lengths.  Full layers (and runs without Omni-Attention) get ``md`` unchanged."""
    om = md.omni
    if om is None or layer_idx >= len(om["pattern"]) or not om["pattern"][layer_idx]:
        return md
    import copy
    v = copy.copy(md)
    v.slot_mapping = om["slot_mapping"]
    if not md.is_prefill:
        v.block_table, v.q_seq_lens, v.max_seq_len, v.q_to_seq = om["block_table"], om["q_seq_lens"], om["max_seq_len"], None
    return v
