"""Qwen2 (dense GQA, omni/models/qwen/qwen2.py:60-566) and Qwen3-MoE-style GQA MoE models."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..layers.common import AttnMetadata, Linear, RMSNorm, SwiGLUMLP, _dtype
from ..layers.gqa import GQAAttention
from ..layers.moe import MoELayer
from ..layers.vocab_parallel import embed, lm_logits, make_embedding, make_lm_head
from .config import ModelConfig


class QwenDecoderLayer(nn.Module):
    def __init__(self, cfg, layer_idx, *, dtype, device, cos_sin, planner=None):
        super().__init__()
        self.quant = cfg.quantization == "fp8_block"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = GQAAttention(cfg, layer_idx, dtype=dtype, device=device, cos_sin=cos_sin)
        self.is_moe = cfg.layer_is_moe(layer_idx)
        if self.is_moe:
            self.mlp = MoELayer(cfg, layer_idx, dtype=dtype, device=device, planner=planner)
        else:
            self.mlp = SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype=dtype,
                                 quant=cfg.quantization if self.quant else "none", device=device)

    def forward_tp(self, h, residual, md, kv_cache, tp, num_valid):
        """The same layer on this rank's token rows, attention sharded by heads (GQAAttention.forward_tp)."""
        if residual is None:
            residual = h.clone()
            n = self.input_layernorm(h, quant=self.quant)
        else:
            n = self.input_layernorm(h, residual=residual, quant=self.quant)
        x, xq = (n[0], (n[1], n[2])) if self.quant else (n, None)
        residual, x = self.self_attn.forward_tp(x, xq, md, kv_cache, residual, self.post_attention_layernorm, tp)
        xq = ops.quant_fp8_block(x) if self.quant else None
        out = self.mlp(x, xq=xq, num_valid=num_valid) if self.is_moe else self.mlp(x, xq=xq)
        return out, residual

    def forward(self, h, residual, md, kv_cache):
        if residual is None:
            residual = h.clone()
            n = self.input_layernorm(h, quant=self.quant)
        else:
            n = self.input_layernorm(h, residual=residual, quant=self.quant)
        x, xq = (n[0], (n[1], n[2])) if self.quant else (n, None)
        a = self.self_attn(x, md, kv_cache, xq=xq)
        n = self.post_attention_layernorm(a, residual=residual, quant=self.quant)
        x, xq = (n[0], (n[1], n[2])) if self.quant else (n, None)
        out = self.mlp(x, xq=xq, num_valid=md.num_valid) if self.is_moe else self.mlp(x, xq=xq)
        return out, residual


class QwenModel(nn.Module):
    def __init__(self, cfg: ModelConfig, *, device=None, planner=None):
        super().__init__()
        self.cfg = cfg
        dtype = _dtype(cfg.dtype)
        self.dtype = dtype
        self.cos_sin = ops.rope_cos_sin_table(cfg.head_dim, min(cfg.max_position_embeddings, 131072), cfg.rope_theta,
                                              cfg.rope_scaling, device=device or "cpu")
        self.embed_tokens = make_embedding(cfg, dtype, device)
        from ..parallel.parallel_state import get_parallel_state
        from ..parallel.pipeline import PipelineStage, PPMissingLayer, layer_range
        ps = get_parallel_state()
        n = cfg.num_hidden_layers
        self.pp = PipelineStage() if ps.pp_size > 1 else None
        self.layer_lo, self.layer_hi = layer_range(n, ps.pp_rank, ps.pp_size) if self.pp else (0, n)
        self.layers = nn.ModuleList([QwenDecoderLayer(cfg, i, dtype=dtype, device=device, cos_sin=self.cos_sin, planner=planner)
                                     if self.layer_lo <= i < self.layer_hi else PPMissingLayer() for i in range(n)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)

    def forward(self, input_ids, md, kv_caches, inputs_embeds=None):
        if self.cfg.attn_tp_size > 1:
            return self._forward_tp(input_ids, md, kv_caches, inputs_embeds)
        pp = self.pp
        if pp is None or pp.is_first:
            h = embed(input_ids, self.embed_tokens.weight) if inputs_embeds is None else inputs_embeds
            residual = None
        else:
            h, residual = pp.recv_intermediate(input_ids.shape[0], self.cfg.hidden_size, self.dtype, input_ids.device)
        for i in range(self.layer_lo, self.layer_hi):
            h, residual = self.layers[i](h, residual, md, kv_caches[i - self.layer_lo])
        if pp is not None and not pp.is_last:
            pp.send_intermediate(h, residual)
            return h
        return self.norm(h, residual=residual)


    def _forward_tp(self, input_ids, md, kv_caches, inputs_embeds=None):
        """Tensor-parallel attention: every rank sees the same batch, works on its block of the (padded) token rows
        between the attention blocks, and gathers the final hidden states so that sampling is identical everywhere."""
        from .deepseek import shard_rows_for_tp
        tp, h, num_valid, T = shard_rows_for_tp(self.cfg, input_ids, md, self.embed_tokens.weight, inputs_embeds)
        residual = None
        for i, layer in enumerate(self.layers):
            h, residual = layer.forward_tp(h, residual, md, kv_caches[i], tp, num_valid)
        out = self.norm(h, residual=residual)
        return tp.all_gather_rows(out.contiguous(), out.shape[0] * tp.world)[:T]


class Qwen2ForCausalLM(nn.Module):
    is_mla = False

    def __init__(self, cfg: ModelConfig, *, device=None, planner=None):
        super().__init__()
        self.cfg = cfg
        self.model = QwenModel(cfg, device=device, planner=planner)
        self.lm_head = None if cfg.tie_word_embeddings else make_lm_head(cfg, self.model.dtype, device)

    @property
    def num_kv_layers(self):
        return self.model.layer_hi - self.model.layer_lo

    def forward(self, input_ids, md, kv_caches, inputs_embeds=None):
        return self.model(input_ids, md, kv_caches, inputs_embeds)

    def compute_logits(self, hidden):
        w = self.lm_head.weight if self.lm_head is not None else self.model.embed_tokens.weight
        return lm_logits(hidden, w, same_rows_everywhere=self.cfg.attn_tp_size > 1)

    def process_weights_after_loading(self):
        pass

    def should_use_eager_mode(self, md):
        return md.is_prefill

    def load_weights(self, weights, planner=None) -> set:
        from ..quantization.loader import WeightLoader
        return WeightLoader(self, self.cfg, planner=planner).load(weights)


Qwen3MoeForCausalLM = Qwen2ForCausalLM
