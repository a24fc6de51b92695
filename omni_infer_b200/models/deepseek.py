"""DeepSeek-V2 / V3 / R1 (MLA + MoE) decoder stack.

Counterpart of the reference's DeepseekDecoderLayer / DeepseekV3Model / DeepseekV3ForCausalLM
(omni/models/deepseek/deepseek_v3.py:139-460, 698-895) and CustomDeepseekV2ForCausalLM
(omni/models/deepseek/deepseek_v2.py:78-685).  One class serves both generations: V2-Lite has no q LoRA
and softmax routing, V3 has q LoRA, sigmoid + bias group-limited routing and block-scaled e4m3 weights.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch
from torch import nn

from .. import ops
from ..layers.common import AttnMetadata, Linear, RMSNorm, SwiGLUMLP, _dtype
from ..layers.mla import MLAAttention
from ..layers.moe import MoELayer
from ..layers.vocab_parallel import embed, lm_logits, make_embedding, make_lm_head
from .config import ModelConfig


class DeepseekDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, *, dtype, device, cos_sin, planner=None, force_moe=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.quant = cfg.quantization == "fp8_block"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = MLAAttention(cfg, layer_idx, dtype=dtype, device=device, cos_sin=cos_sin)
        is_moe = cfg.layer_is_moe(layer_idx) if force_moe is None else force_moe
        if is_moe:
            self.mlp = MoELayer(cfg, layer_idx, dtype=dtype, device=device, planner=planner)
        else:
            q = cfg.quantization if self.quant else "none"
            if cfg.dense_mlp_tp_size > 1 and cfg.attn_tp_size == 1:
                from ..layers.linear import ParallelSwiGLUMLP
                self.mlp = ParallelSwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype=dtype, quant=q, device=device)
            else:
                self.mlp = SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype=dtype, quant=q, device=device)
        self.is_moe = is_moe

    def forward_tp(self, h, residual, md: AttnMetadata, kv_cache, tp, num_valid):
        """Same layer on this rank's token rows, attention sharded by heads (see MLAAttention.forward_tp)."""
        if residual is None:
            residual = h.clone()
            n = self.input_layernorm(h, quant=self.quant)
        else:
            n = self.input_layernorm(h, residual=residual, quant=self.quant)
        x, xq = (n[0], (n[1], n[2])) if self.quant else (n, None)
        residual, x = self.self_attn.forward_tp(x, xq, md, kv_cache, residual, self.post_attention_layernorm, tp)
        xq = ops.quant_fp8_block(x) if self.quant else None
        if self.is_moe:
            out = self.mlp(x, xq=xq, num_valid=num_valid)
        else:
            out = self.mlp(x, xq=xq)
        return out, residual

    def forward(self, h, residual, md: AttnMetadata, kv_cache):
        if residual is None:
            residual = h.clone()
            n = self.input_layernorm(h, quant=self.quant)
        else:
            n = self.input_layernorm(h, residual=residual, quant=self.quant)
        x, xq = (n[0], (n[1], n[2])) if self.quant else (n, None)
        a = self.self_attn(x, md, kv_cache, xq=xq)
        n = self.post_attention_layernorm(a, residual=residual, quant=self.quant)
        x, xq = (n[0], (n[1], n[2])) if self.quant else (n, None)
        if self.is_moe:
            out = self.mlp(x, xq=xq, num_valid=md.num_valid)
        else:
            out = self.mlp(x, xq=xq)
        return out, residual


def shard_rows_for_tp(cfg, input_ids, md, embed_weight, inputs_embeds=None):
    """This rank's block of the token rows, padded so that every rank has the same number (a multiple of four:
    activation-scale rows are copied 16 bytes at a time).  Returns (tp context, rows [rpr, hidden], number of
    valid rows among them as a device tensor, real row count)."""
    from ..parallel.parallel_state import get_parallel_state
    tp = get_parallel_state().tp_fused
    assert tp is not None, "tensor-parallel attention needs the runner to set up the TP context first"
    W, r = tp.world, tp.rank
    T = input_ids.shape[0] if inputs_embeds is None else inputs_embeds.shape[0]
    step = W * 4
    Tp = (T + step - 1) // step * step
    rpr = Tp // W
    lo, hi = r * rpr, min(T, (r + 1) * rpr)
    if inputs_embeds is None:
        ids = input_ids[lo:hi] if hi > lo else input_ids[:0]
        h = embed(ids, embed_weight)
    else:
        h = inputs_embeds[lo:hi] if hi > lo else inputs_embeds[:0]
    if h.shape[0] < rpr:
        h = torch.cat([h, h.new_zeros(rpr - h.shape[0], h.shape[1])], 0)
    dev = h.device
    if md.num_valid is not None:
        nv = (md.num_valid[:1].to(torch.int32) - lo).clamp(0, rpr)
    else:
        nv = torch.tensor([max(0, hi - lo)], dtype=torch.int32, device=dev) if Tp != T else None
    return tp, h.contiguous(), nv, T


class DeepseekModel(nn.Module):
    def __init__(self, cfg: ModelConfig, *, device=None, planner=None, num_layers: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        dtype = _dtype(cfg.dtype)
        self.dtype = dtype
        self.cos_sin = ops.rope_cos_sin_table(cfg.qk_rope_head_dim, min(cfg.max_position_embeddings, 163840),
                                              cfg.rope_theta, cfg.rope_scaling, device=device or "cpu")
        self.embed_tokens = make_embedding(cfg, dtype, device)
        n = cfg.num_hidden_layers if num_layers is None else num_layers
        # pipeline parallelism: this stage builds its own block of layers, placeholders keep the indices of the others
        from ..parallel.parallel_state import get_parallel_state
        from ..parallel.pipeline import PipelineStage, PPMissingLayer, layer_range
        ps = get_parallel_state()
        self.pp = PipelineStage() if ps.pp_size > 1 else None
        self.layer_lo, self.layer_hi = layer_range(n, ps.pp_rank, ps.pp_size) if self.pp else (0, n)
        self.layers = nn.ModuleList([
            DeepseekDecoderLayer(cfg, i, dtype=dtype, device=device, cos_sin=self.cos_sin, planner=planner)
            if self.layer_lo <= i < self.layer_hi else PPMissingLayer() for i in range(n)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)

    def forward(self, input_ids, md: AttnMetadata, kv_caches, inputs_embeds=None):
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
            pp.send_intermediate(h, residual)      # the next stage goes on from here; this stage has no logits
            return h
        return self.norm(h, residual=residual)

    def _forward_tp(self, input_ids, md: AttnMetadata, kv_caches, inputs_embeds=None):
        """Tensor-parallel attention: every rank sees the same batch, works on its block of the (padded) token rows
        between the attention blocks, and gathers the final hidden states so that sampling is identical everywhere."""
        from ..parallel.parallel_state import get_parallel_state
        tp, h, num_valid, T = shard_rows_for_tp(self.cfg, input_ids, md, self.embed_tokens.weight, inputs_embeds)
        residual = None
        for i, layer in enumerate(self.layers):
            h, residual = layer.forward_tp(h, residual, md, kv_caches[i], tp, num_valid)
        out = self.norm(h, residual=residual)
        return tp.all_gather_rows(out.contiguous(), out.shape[0] * tp.world)[:T]


class DeepseekV3ForCausalLM(nn.Module):
    """Returns hidden states from ``forward`` and logits from ``compute_logits`` (the model runner keeps
    the hidden states for the MTP drafters)."""
    is_mla = True

    def __init__(self, cfg: ModelConfig, *, device=None, planner=None):
        super().__init__()
        self.cfg = cfg
        self.model = DeepseekModel(cfg, device=device, planner=planner)
        dtype = self.model.dtype
        if cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = make_lm_head(cfg, dtype, device)

    @property
    def num_kv_layers(self) -> int:
        return self.model.layer_hi - self.model.layer_lo

    def forward(self, input_ids, md: AttnMetadata, kv_caches, inputs_embeds=None):
        return self.model(input_ids, md, kv_caches, inputs_embeds)

    def compute_logits(self, hidden):
        w = self.lm_head.weight if self.lm_head is not None else self.model.embed_tokens.weight
        return lm_logits(hidden, w, same_rows_everywhere=self.cfg.attn_tp_size > 1)

    def process_weights_after_loading(self):
        for layer in self.model.layers[self.model.layer_lo:self.model.layer_hi]:
            layer.self_attn.process_weights_after_loading()

    def should_use_eager_mode(self, md: AttnMetadata) -> bool:
        """Prefill runs eagerly, decode-only steps replay CUDA graphs
        (omni/models/deepseek/deepseek_v3.py:897-908)."""
        return md.is_prefill

    # ------------------------------------------------------------------ checkpoint loading
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]], planner=None) -> set:
        from ..quantization.loader import WeightLoader
        return WeightLoader(self, self.cfg, planner=planner).load(weights)


DeepseekV2ForCausalLM = DeepseekV3ForCausalLM
