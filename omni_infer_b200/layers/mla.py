"""Multi-head Latent Attention (DeepSeek-V2/V3).

Prefill runs the non-absorbed form (q 192-wide, k = [k_nope | k_pe], v 128-wide, causal varlen); decode
runs the absorbed form over the paged latent cache: ``q_abs = q_nope @ W_UK``, scores against the
576-wide cache rows, output in latent space, then ``@ W_UV`` and o_proj
(omni/models/common/layers/attention/deepseek_mla.py:209-235, 269-410, 412-661).
The latent cache of a layer is one tensor [blocks, block_size, kv_lora + rope]."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops

from .common import AttnMetadata, Linear, RMSNorm


class MLAAttention(nn.Module):
    def __init__(self, cfg, layer_idx: int, *, dtype, device=None, cos_sin=None):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        H_all = cfg.num_attention_heads
        self.tp_world, self.tp_rank = int(getattr(cfg, "attn_tp_size", 1)), int(getattr(cfg, "attn_tp_rank", 0))
        assert H_all % self.tp_world == 0, "attention heads must divide over the tensor-parallel ranks"
        H = H_all // self.tp_world          # heads computed by this rank
        self.H, self.H_all = H, H_all
        self.nope, self.rope, self.vd = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.kvl = cfg.kv_lora_rank
        self.qk = self.nope + self.rope
        self.scale = cfg.softmax_scale
        quant = cfg.quantization if cfg.quantization == "fp8_block" else "none"
        self.quant = quant
        hs = cfg.hidden_size
        self.q_lora = cfg.q_lora_rank
        if self.q_lora:
            # merged q_a + kv_a projection: both read the same normalised hidden state
            self.fused_qkv_a_proj = Linear(hs, self.q_lora + self.kvl + self.rope, dtype=dtype, quant=quant, device=device)
            self.q_a_layernorm = RMSNorm(self.q_lora, cfg.rms_norm_eps, dtype, device)
            self.q_b_proj = Linear(self.q_lora, H * self.qk, dtype=dtype, quant=quant, device=device)
        else:
            self.fused_qkv_a_proj = Linear(hs, H * self.qk + self.kvl + self.rope, dtype=dtype, quant=quant, device=device)
        self.kv_a_layernorm = RMSNorm(self.kvl, cfg.rms_norm_eps, dtype, device)
        # kept unquantised: the absorbed decode path multiplies activations by slices of it
        self.kv_b_proj = Linear(self.kvl, H * (self.nope + self.vd), dtype=dtype, quant="none", device=device)
        if getattr(cfg, "o_proj_tp_size", 1) > 1 and self.tp_world == 1:
            # attention stays data parallel, o_proj is sharded over the o_proj_tp sub-group
            from ..parallel import get_parallel_state
            from .linear import DP2TPRowParallelLinear
            self.o_proj = DP2TPRowParallelLinear(H * self.vd, hs, get_parallel_state().group("o_proj_tp"), dtype=dtype,
                                                 quant=quant, device=device)
        else:
            self.o_proj = Linear(H * self.vd, hs, dtype=dtype, quant=quant, device=device)
        self.cos_sin = cos_sin
        if self.tp_world > 1:
            self._mark_tp_shards()
        self.w_uk = None   # [H, kvl, nope]   (N = kvl, K = nope)
        self.w_uv = None   # [H, vd, kvl]     (N = vd,  K = kvl)

    def _mark_tp_shards(self):
        """Tell the weight loaders which slice of the full tensor each sharded parameter holds: q / kv_b rows by
        head (column parallel), o_proj columns by head (row parallel); the kv_a rows are replicated."""
        r, Hl, Ha = self.tp_rank, self.H, self.H_all

        def rows(unit):
            return lambda full: full[r * Hl * unit:(r + 1) * Hl * unit]

        def mark(lin, fn, scale_fn=None, full=None):
            lin.weight.tp_slice_fn = fn
            lin.weight.tp_full_shape = full
            if lin.weight_scale is not None:
                lin.weight_scale.tp_slice_fn = scale_fn

        def srows(unit):   # the same row slice in units of 128-row scale blocks
            assert (Hl * unit) % 128 == 0, "fp8 shards must be aligned to the 128x128 scale blocks"
            return lambda full: full[r * Hl * unit // 128:(r + 1) * Hl * unit // 128]

        fp8 = self.quant == "fp8_block"
        if self.q_lora:
            mark(self.q_b_proj, rows(self.qk), srows(self.qk) if fp8 else None, full=(Ha * self.qk, self.q_lora))
        else:
            qk, tail0 = self.qk, Ha * self.qk
            assert not fp8, "fp8 without q LoRA is not sharded here"
            mark(self.fused_qkv_a_proj, lambda full: torch.cat([full[r * Hl * qk:(r + 1) * Hl * qk], full[tail0:]], 0),
                 full=(Ha * qk + self.kvl + self.rope, self.cfg.hidden_size))
        mark(self.kv_b_proj, rows(self.nope + self.vd), full=(Ha * (self.nope + self.vd), self.kvl))
        vd = self.vd
        if fp8:
            assert (Hl * vd) % 128 == 0
        mark(self.o_proj, lambda full: full[:, r * Hl * vd:(r + 1) * Hl * vd].contiguous(),
             (lambda full: full[:, r * Hl * vd // 128:(r + 1) * Hl * vd // 128].contiguous()) if fp8 else None,
             full=(self.cfg.hidden_size, Ha * vd))

    def process_weights_after_loading(self):
        w = self.kv_b_proj.weight.view(self.H, self.nope + self.vd, self.kvl)
        self.w_uk = w[:, : self.nope, :].transpose(1, 2).contiguous()
        self.w_uv = w[:, self.nope:, :].contiguous()

    # ------------------------------------------------------------------ projections
    def _project(self, x, xq, md: AttnMetadata, kv_cache, decode: bool):
        T = x.shape[0]
        H = self.H
        a = self.fused_qkv_a_proj(x, xq=xq)
        if self.q_lora:
            q_a = a[:, : self.q_lora]
            latent = a[:, self.q_lora:]
            if self.quant == "fp8_block":
                _, qa_q, qa_s = self.q_a_layernorm(q_a, quant=True)
                q = self.q_b_proj(None, xq=(qa_q, qa_s))
            else:
                q = self.q_b_proj(self.q_a_layernorm(q_a))
        else:
            q = a[:, : H * self.qk].contiguous()
            latent = a[:, H * self.qk:]
        q = q.view(T, H, self.qk)
        return q, latent

    # ------------------------------------------------------------------ forward
    def forward(self, x, md: AttnMetadata, kv_cache, xq=None):
        md = _omni_view(md, self.layer_idx)
        if md.is_prefill:
            return self._forward_prefill(x, xq, md, kv_cache)
        return self._forward_decode(x, xq, md, kv_cache)

    def _forward_prefill(self, x, xq, md, kv_cache):
        T, H = x.shape[0], self.H
        q, latent = self._project(x, xq, md, kv_cache, decode=False)
        lat = ops.mla_kv_rope_cache(latent, self.kv_a_layernorm.weight, self.kv_a_layernorm.eps, self.cos_sin,
                                    md.positions, md.slot_mapping, kv_cache, q=q, q_rope_off=self.nope,
                                    want_latent=True)
        if md.kv_gather_slots is not None:
            # prefix-cache / chunked prefill: attend over the whole cached context of each request
            lat = kv_cache.view(-1, kv_cache.shape[-1])[md.kv_gather_slots, : self.kvl + self.rope]
        kv = self.kv_b_proj(lat[:, : self.kvl].contiguous() if not lat.is_cuda else lat[:, : self.kvl])
        o = ops.attention.mla_prefill(q, kv, lat, H, self.nope, self.rope, self.vd, md.cu_q, md.cu_k, self.scale,
                                      md.max_q, md.max_k)
        return self.o_proj(o.reshape(T, H * self.vd))

    def _forward_decode(self, x, xq, md, kv_cache):
        T, H = x.shape[0], self.H
        q, latent = self._project(x, xq, md, kv_cache, decode=True)
        q_abs = torch.empty(T, H, self.kvl + self.rope, dtype=x.dtype, device=x.device)
        ops.bmm_heads(q[:, :, : self.nope], self.w_uk, out=q_abs)
        ops.mla_kv_rope_cache(latent, self.kv_a_layernorm.weight, self.kv_a_layernorm.eps, self.cos_sin, md.positions,
                              md.slot_mapping, kv_cache, q=q, q_rope_off=self.nope, q_out=q_abs, q_out_off=self.kvl)
        o_lat = ops.mla_decode(q_abs, kv_cache, md.block_table, md.q_seq_lens, self.scale, q_to_seq=md.q_to_seq,
                               max_seq_len=md.max_seq_len, kv_lora=self.kvl)
        o = ops.bmm_heads(o_lat, self.w_uv)
        return self.o_proj(o.reshape(T, H * self.vd))


    # ------------------------------------------------------------------ tensor-parallel form
    def forward_tp(self, x_shard, xq_shard, md: AttnMetadata, kv_cache, residual_shard, post_norm, tp):
        """Heads sharded over the ranks, hidden states sharded by token rows outside the attention block.
        ``x_shard`` [rpr, hidden] are this rank's rows of the normalised input (``xq_shard`` its e4m3 form).  The
        row all-gather is fused into the first projection and o_proj into the reduce-scatter, which also adds the
        residual and applies ``post_norm``.  Returns (new residual rows, normalised rows)
        (omni/models/common/layers/attention/deepseek_mla.py:437-470)."""
        md = _omni_view(md, self.layer_idx)
        rpr = x_shard.shape[0]
        Tp = rpr * tp.world                      # padded token rows of the step
        T = md.positions.shape[0]                # real token rows (<= Tp)
        H = self.H
        lin = self.fused_qkv_a_proj
        if self.quant == "fp8_block":
            a, _, _ = tp.allgather_gemm(xq_shard[0], lin.weight, total_rows=Tp, w_scale=lin.weight_scale,
                                        x_scale_shard=xq_shard[1])
        else:
            a, _, _ = tp.allgather_gemm(x_shard, lin.weight, total_rows=Tp)
        a = a[:T]
        if self.q_lora:
            q_a, latent = a[:, : self.q_lora], a[:, self.q_lora:]
            if self.quant == "fp8_block":
                _, qa_q, qa_s = self.q_a_layernorm(q_a, quant=True)
                q = self.q_b_proj(None, xq=(qa_q, qa_s))
            else:
                q = self.q_b_proj(self.q_a_layernorm(q_a))
        else:
            q, latent = a[:, : H * self.qk].contiguous(), a[:, H * self.qk:]
        q = q.view(T, H, self.qk)
        if md.is_prefill:
            lat = ops.mla_kv_rope_cache(latent, self.kv_a_layernorm.weight, self.kv_a_layernorm.eps, self.cos_sin,
                                        md.positions, md.slot_mapping, kv_cache, q=q, q_rope_off=self.nope, want_latent=True)
            if md.kv_gather_slots is not None:
                lat = kv_cache.view(-1, kv_cache.shape[-1])[md.kv_gather_slots, : self.kvl + self.rope]
            kv = self.kv_b_proj(lat[:, : self.kvl])
            o = ops.attention.mla_prefill(q, kv, lat, H, self.nope, self.rope, self.vd, md.cu_q, md.cu_k, self.scale,
                                          md.max_q, md.max_k)
        else:
            q_abs = torch.empty(T, H, self.kvl + self.rope, dtype=x_shard.dtype, device=x_shard.device)
            ops.bmm_heads(q[:, :, : self.nope], self.w_uk, out=q_abs)
            ops.mla_kv_rope_cache(latent, self.kv_a_layernorm.weight, self.kv_a_layernorm.eps, self.cos_sin, md.positions,
                                  md.slot_mapping, kv_cache, q=q, q_rope_off=self.nope, q_out=q_abs, q_out_off=self.kvl)
            o_lat = ops.mla_decode(q_abs, kv_cache, md.block_table, md.q_seq_lens, self.scale, q_to_seq=md.q_to_seq,
                                   max_seq_len=md.max_seq_len, kv_lora=self.kvl)
            o = ops.bmm_heads(o_lat, self.w_uv)
        o = o.reshape(T, H * self.vd)
        if T < Tp:   # padding rows contribute zeros to the sum
            o = torch.cat([o, o.new_zeros(Tp - T, o.shape[1])], 0)
        op = self.o_proj
        if self.quant == "fp8_block":
            oq, os_ = ops.quant_fp8_block(o)
            return tp.gemm_reduce_scatter(oq, op.weight, w_scale=op.weight_scale, x_scale=os_, residual=residual_shard,
                                          norm_weight=post_norm.weight, eps=post_norm.eps)
        return tp.gemm_reduce_scatter(o, op.weight, residual=residual_shard, norm_weight=post_norm.weight, eps=post_norm.eps)


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
