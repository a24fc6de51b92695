"""Grouped-query attention (Qwen2 / Qwen3-MoE) over a paged K/V cache
(reference backend: omni/models/common/layers/attention/backend/attention.py:507-702)."""
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
        self.Hq, self.Hkv, self.D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        quant = cfg.quantization if cfg.quantization == "fp8_block" else "none"
        self.qkv_proj = Linear(cfg.hidden_size, (self.Hq + 2 * self.Hkv) * self.D, dtype=dtype, quant=quant,
                               bias=cfg.attention_bias, device=device)
        self.o_proj = Linear(self.Hq * self.D, cfg.hidden_size, dtype=dtype, quant=quant, device=device)
        self.q_norm = RMSNorm(self.D, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.k_norm = RMSNorm(self.D, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.scale = self.D ** -0.5
        self.cos_sin = cos_sin

    def process_weights_after_loading(self):
        pass

    def forward(self, x, md: AttnMetadata, kv_cache, xq=None):
        md = _omni_view(md, self.layer_idx)
        T = x.shape[0]
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        k_cache, v_cache = kv_cache
        qkv = self.qkv_proj(x, xq=xq)
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
        return self.o_proj(o.reshape(T, Hq * D))


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
