"""DeepSeek multi-token-prediction drafter (omni/models/deepseek/deepseek_mtp.py:40-129, 173-286).

One drafter = enorm + hnorm + eh_proj (2H -> H) + one decoder layer (checkpoint layer index
``num_hidden_layers + i``) + shared-head norm; embedding and LM head are shared with the main model.
``forward(tokens, previous_hidden)`` -> hidden; ``compute_logits`` through the shared head."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..layers.vocab_parallel import embed
from ..layers.common import AttnMetadata, Linear, RMSNorm, _dtype
from .config import ModelConfig
from .deepseek import DeepseekDecoderLayer


class DeepseekV3MTP(nn.Module):
    is_mla = True

    def __init__(self, cfg: ModelConfig, main_model, mtp_index: int = 0, *, device=None, planner=None):
        super().__init__()
        self.cfg = cfg
        dtype = _dtype(cfg.dtype)
        self.mtp_index = mtp_index
        self.layer_idx = cfg.num_hidden_layers + mtp_index
        H = cfg.hidden_size
        self.enorm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        self.hnorm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        self.eh_proj = Linear(2 * H, H, dtype=dtype, device=device)
        self.decoder = DeepseekDecoderLayer(cfg, self.layer_idx, dtype=dtype, device=device,
                                            cos_sin=main_model.model.cos_sin, planner=None,
                                            force_moe=cfg.is_moe)
        self.shared_head_norm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        # shared with the main model (not registered as sub-modules: no double ownership of the tensors)
        object.__setattr__(self, "_main", main_model)

    @property
    def num_kv_layers(self) -> int:
        return 1

    def forward(self, input_ids, md: AttnMetadata, kv_caches, previous_hidden_states):
        emb = embed(input_ids, self._main.model.embed_tokens.weight)
        x = torch.cat([self.enorm(emb), self.hnorm(previous_hidden_states)], dim=-1)
        h = self.eh_proj(x)
        if self.cfg.attn_tp_size > 1:
            # tensor-parallel attention: the drafter layer works on this rank's block of the rows like the main stack
            from ..parallel.parallel_state import get_parallel_state
            from .deepseek import shard_rows_for_tp
            tp, hs, nv, T = shard_rows_for_tp(self.cfg, input_ids, md, None, inputs_embeds=h)
            hs, residual = self.decoder.forward_tp(hs, None, md, kv_caches[0], tp, nv)
            out = self.shared_head_norm(hs, residual=residual)
            return tp.all_gather_rows(out.contiguous(), out.shape[0] * tp.world)[:T]
        h, residual = self.decoder(h, None, md, kv_caches[0])
        return self.shared_head_norm(h, residual=residual)

    def compute_logits(self, hidden):
        return self._main.compute_logits(hidden)

    def process_weights_after_loading(self):
        self.decoder.self_attn.process_weights_after_loading()

    def load_weights(self, weights, planner=None) -> set:
        from ..quantization.loader import WeightLoader
        return WeightLoader(self, self.cfg, planner=planner, mtp_layer=self.layer_idx).load(weights)


class DeepSeekMTPModel(DeepseekV3MTP):
    """First drafter (layer ``num_hidden_layers``)."""


class DeepSeekMTPModelDuo(DeepseekV3MTP):
    def __init__(self, cfg, main_model, **kw):
        super().__init__(cfg, main_model, mtp_index=1, **kw)


class DeepSeekMTPModelTres(DeepseekV3MTP):
    def __init__(self, cfg, main_model, **kw):
        super().__init__(cfg, main_model, mtp_index=2, **kw)
