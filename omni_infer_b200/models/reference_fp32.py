"""Plain-PyTorch fp32 oracle for the DeepSeek-style MLA + MoE models.

Deliberately naive and independent of the engine: no KV cache (the whole sequence is recomputed for
every generated token), non-absorbed attention with explicit per-head K/V, a dense loop over experts,
straightforward RMSNorm / RoPE.  It reads the weights of an engine model through ``state_dict`` and is
the golden reference for end-to-end greedy tokens and for the fused kernels' numerics."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from ..ops.gemm import FP8, dequant_weight_ref
from .config import ModelConfig


def _w(sd, name):
    w = sd[name]
    if w.dtype == FP8:
        w = dequant_weight_ref(w, sd[name + "_scale"])
    return w.float().cpu()


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope_interleaved(x, cos, sin):
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)


class ReferenceDeepseek:
    def __init__(self, cfg: ModelConfig, state_dict: dict, prefix: str = ""):
        self.cfg, self.sd, self.prefix = cfg, state_dict, prefix
        self.cos_sin = ops.rope_cos_sin_table(cfg.qk_rope_head_dim, min(cfg.max_position_embeddings, 8192),
                                              cfg.rope_theta, cfg.rope_scaling)

    # ------------------------------------------------------------------ pieces
    def _attn(self, x, p):
        cfg, sd = self.cfg, self.sd
        L, H = x.shape[0], cfg.num_attention_heads
        nope, rope, vd, kvl = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        a = x @ _w(sd, p + "fused_qkv_a_proj.weight").t()
        if cfg.q_lora_rank:
            q_a, latent = a[:, : cfg.q_lora_rank], a[:, cfg.q_lora_rank:]
            q = _rms(q_a, _w(sd, p + "q_a_layernorm.weight"), cfg.rms_norm_eps) @ _w(sd, p + "q_b_proj.weight").t()
        else:
            q, latent = a[:, : H * (nope + rope)], a[:, H * (nope + rope):]
        q = q.view(L, H, nope + rope)
        c_kv = _rms(latent[:, :kvl], _w(sd, p + "kv_a_layernorm.weight"), cfg.rms_norm_eps)
        cs = self.cos_sin[:L]
        cos, sin = cs[:, : rope // 2], cs[:, rope // 2:]
        k_pe = _rope_interleaved(latent[:, kvl:], cos, sin)
        q_pe = _rope_interleaved(q[..., nope:], cos[:, None], sin[:, None])
        kv = (c_kv @ _w(sd, p + "kv_b_proj.weight").t()).view(L, H, nope + vd)
        k = torch.cat([kv[..., :nope], k_pe[:, None].expand(L, H, rope)], dim=-1)
        qq = torch.cat([q[..., :nope], q_pe], dim=-1)
        s = torch.einsum("ihd,jhd->hij", qq, k) * cfg.softmax_scale
        s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), kv[..., nope:]).reshape(L, H * vd)
        return o @ _w(sd, p + "o_proj.weight").t()

    def _mlp(self, x, p):
        g = x @ _w(self.sd, p + "gate_up_proj.weight").t()
        i = g.shape[-1] // 2
        return (F.silu(g[:, :i]) * g[:, i:]) @ _w(self.sd, p + "down_proj.weight").t()

    def _moe(self, x, p):
        cfg, sd = self.cfg, self.sd
        logits = x @ _w(sd, p + "gate.weight").t()
        bias = sd.get(p + "gate.e_score_correction_bias")
        if cfg.topk_method == "noaux_tc":
            kw = dict(mode="sigmoid", bias=bias.float().cpu(), n_group=cfg.n_group, topk_group=cfg.topk_group,
                      group_mode="top2sum", renorm=cfg.norm_topk_prob, scale=cfg.routed_scaling_factor)
        elif cfg.topk_method == "group_limited_greedy":
            kw = dict(mode=cfg.scoring_func, n_group=cfg.n_group, topk_group=cfg.topk_group, group_mode="max",
                      renorm=cfg.norm_topk_prob, scale=cfg.routed_scaling_factor)
        else:
            kw = dict(mode=cfg.scoring_func, renorm=cfg.norm_topk_prob, scale=cfg.routed_scaling_factor)
        ids, w = ops.router_topk_ref(logits, cfg.num_experts_per_tok, **kw)
        w13, w2 = _w(sd, p + "w13"), _w(sd, p + "w2")
        out = torch.zeros_like(x)
        I = cfg.moe_intermediate_size
        for t in range(x.shape[0]):
            for j in range(ids.shape[1]):
                e = int(ids[t, j])
                g = w13[e] @ x[t]
                out[t] += w[t, j] * (w2[e] @ (F.silu(g[:I]) * g[I:]))
        if cfg.n_shared_experts:
            out = out + self._mlp(x, p + "shared_experts.")
        return out

    # ------------------------------------------------------------------ whole model
    def hidden(self, token_ids: list) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        h = _w(sd, "model.embed_tokens.weight")[torch.tensor(token_ids)]
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            x = _rms(h, _w(sd, p + "input_layernorm.weight"), cfg.rms_norm_eps)
            h = h + self._attn(x, p + "self_attn.")
            x = _rms(h, _w(sd, p + "post_attention_layernorm.weight"), cfg.rms_norm_eps)
            h = h + (self._moe(x, p + "mlp.") if cfg.layer_is_moe(i) else self._mlp(x, p + "mlp."))
        return _rms(h, _w(sd, "model.norm.weight"), cfg.rms_norm_eps)

    def logits(self, token_ids: list) -> torch.Tensor:
        h = self.hidden(token_ids)
        head = "lm_head.weight" if "lm_head.weight" in self.sd else "model.embed_tokens.weight"
        return h @ _w(self.sd, head).t()

    def greedy(self, prompt: list, max_tokens: int) -> list:
        toks = list(prompt)
        out = []
        for _ in range(max_tokens):
            t = int(self.logits(toks)[-1].argmax())
            out.append(t)
            toks.append(t)
        return out


class ReferenceQwen(ReferenceDeepseek):
    """The same naive recomputation for the GQA models (Qwen2: dense, biased qkv; Qwen3-MoE: per-head q/k RMSNorm,
    routed experts without a shared one).  Only the attention differs: explicit per-head K/V repeated over the query
    groups, rotate-half RoPE."""

    def __init__(self, cfg: ModelConfig, state_dict: dict, prefix: str = ""):
        self.cfg, self.sd, self.prefix = cfg, state_dict, prefix
        self.cos_sin = ops.rope_cos_sin_table(cfg.head_dim, min(cfg.max_position_embeddings, 8192), cfg.rope_theta,
                                              cfg.rope_scaling)

    def _attn(self, x, p):
        cfg, sd = self.cfg, self.sd
        L, Hq, Hkv, D = x.shape[0], cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        qkv = x @ _w(sd, p + "qkv_proj.weight").t()
        if p + "qkv_proj.bias" in sd:
            qkv = qkv + sd[p + "qkv_proj.bias"].float().cpu()
        qkv = qkv.view(L, Hq + 2 * Hkv, D)
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
        if cfg.qk_norm:
            q = _rms(q, _w(sd, p + "q_norm.weight"), cfg.rms_norm_eps)
            k = _rms(k, _w(sd, p + "k_norm.weight"), cfg.rms_norm_eps)
        cs = self.cos_sin[:L]
        cos, sin = cs[:, None, : D // 2], cs[:, None, D // 2:]

        def rot(t):
            a, b = t[..., : D // 2], t[..., D // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

        q, k = rot(q), rot(k)
        rep = Hq // Hkv
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        s = torch.einsum("ihd,jhd->hij", q, k) * D ** -0.5
        s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v).reshape(L, Hq * D)
        return o @ _w(sd, p + "o_proj.weight").t()


def reference_for(cfg: ModelConfig, state_dict: dict):
    return ReferenceDeepseek(cfg, state_dict) if cfg.use_mla else ReferenceQwen(cfg, state_dict)
