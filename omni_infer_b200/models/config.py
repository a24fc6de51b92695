"""Architecture description shared by all model families (DeepSeek-V2/V3 MLA+MoE, MTP drafters,
Qwen2 dense GQA, Qwen3-MoE GQA) plus the named configurations used by the benchmarks."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Optional


@dataclass
class ModelConfig:
    architecture: str = "DeepseekV3ForCausalLM"
    # tensor-parallel attention: heads sharded over attn_tp_size ranks, hidden states sharded by token rows between
    # layers (set by the model runner; 1 = every rank runs whole attention layers on its own requests)
    attn_tp_size: int = 1
    attn_tp_rank: int = 0
    # sub-group sharding while attention is data parallel: the dense MLP layers and the shared expert over the
    # ``mlp_tp`` group, o_proj over the ``o_proj_tp`` group (set by the worker from the engine configuration)
    dense_mlp_tp_size: int = 1
    o_proj_tp_size: int = 1
    # dedicated shared-expert ranks: the first N ranks of the expert-parallel group hold only the shared expert, the routed
    # experts are spread over the others (0 = the shared expert runs on every rank beside its routed experts)
    shared_expert_ranks: int = 0
    # vocabulary-parallel embedding table and LM head: each rank holds ceil(vocab / size) rows (set by the model runner)
    vocab_parallel_size: int = 1
    vocab_parallel_rank: int = 0
    # benchmark aid: {"s": 1.2, "strength": 6.0, "seed": 0} adds a fixed Zipf-shaped bias to every router's logits so that
    # expert popularity is skewed (load-balance stress); None = the router as trained
    router_skew: Optional[dict] = None
    vocab_size: int = 1024
    hidden_size: int = 256
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 4
    head_dim: int = 64                       # GQA models
    # MLA
    use_mla: bool = True
    q_lora_rank: int = 0
    kv_lora_rank: int = 64
    qk_nope_head_dim: int = 32
    qk_rope_head_dim: int = 16
    v_head_dim: int = 32
    # MLP / MoE
    intermediate_size: int = 512
    moe_intermediate_size: int = 128
    n_routed_experts: int = 0
    n_shared_experts: int = 0
    num_experts_per_tok: int = 0
    first_k_dense_replace: int = 0
    moe_layer_freq: int = 1
    scoring_func: str = "softmax"            # softmax | sigmoid
    topk_method: str = "greedy"              # greedy | group_limited_greedy | noaux_tc
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = False
    routed_scaling_factor: float = 1.0
    # misc
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    qk_norm: bool = False                    # Qwen3 per-head q/k RMSNorm
    attention_bias: bool = False             # Qwen2 qkv bias
    num_nextn_predict_layers: int = 0        # MTP layers stored after the main stack
    quantization: str = "none"               # none | fp8_block | w8a8_int8
    dtype: str = "bfloat16"
    name: str = ""

    # ---- derived
    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def is_moe(self) -> bool:
        return self.n_routed_experts > 0

    def layer_is_moe(self, layer_idx: int) -> bool:
        return (self.is_moe and layer_idx >= self.first_k_dense_replace
                and layer_idx % self.moe_layer_freq == 0)

    @property
    def softmax_scale(self) -> float:
        """MLA: (nope+rope)^-0.5 * mscale^2 with the YaRN mscale_all_dim correction
        (omni/models/common/layers/attention/deepseek_mla.py:43-48, 173-177)."""
        import math

        d = self.qk_head_dim if self.use_mla else self.head_dim
        scale = d ** -0.5
        rs = self.rope_scaling
        if self.use_mla and rs and rs.get("factor", 1.0) > 1.0 and rs.get("mscale_all_dim", 0):
            m = 0.1 * rs["mscale_all_dim"] * math.log(rs["factor"]) + 1.0
            scale = scale * m * m
        return scale

    def kv_bytes_per_token(self, elem_bytes: int = 2) -> int:
        if self.use_mla:
            return (self.kv_lora_rank + self.qk_rope_head_dim) * elem_bytes
        return 2 * self.local_kv_heads * self.head_dim * elem_bytes

    @property
    def local_kv_heads(self) -> int:
        """K/V heads cached by one rank (all of them unless attention runs tensor parallel)."""
        return max(1, self.num_key_value_heads // max(1, self.attn_tp_size))

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_hf_dict(cls, d: dict[str, Any]) -> "ModelConfig":
        arch = (d.get("architectures") or [d.get("architecture", "DeepseekV3ForCausalLM")])[0]
        c = cls(architecture=arch)
        for k in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                  "moe_intermediate_size", "n_routed_experts", "n_shared_experts", "num_experts_per_tok",
                  "first_k_dense_replace", "moe_layer_freq", "scoring_func", "topk_method", "n_group", "topk_group",
                  "norm_topk_prob", "routed_scaling_factor", "rms_norm_eps", "rope_theta", "rope_scaling",
                  "max_position_embeddings", "tie_word_embeddings", "kv_lora_rank", "qk_nope_head_dim",
                  "qk_rope_head_dim", "v_head_dim", "num_nextn_predict_layers"):
            if k in d and d[k] is not None:
                setattr(c, k, d[k])
        c.q_lora_rank = d.get("q_lora_rank") or 0
        c.num_key_value_heads = d.get("num_key_value_heads", c.num_attention_heads)
        c.use_mla = "Deepseek" in arch
        if not c.use_mla:
            c.head_dim = d.get("head_dim", c.hidden_size // c.num_attention_heads)
            c.attention_bias = "Qwen2" in arch
            c.qk_norm = "Qwen3" in arch
            if "num_experts" in d:   # Qwen MoE naming
                c.n_routed_experts = d["num_experts"]
                c.num_experts_per_tok = d.get("num_experts_per_tok", 8)
                c.moe_intermediate_size = d.get("moe_intermediate_size", c.moe_intermediate_size)
                c.norm_topk_prob = d.get("norm_topk_prob", True)
        qc = d.get("quantization_config") or {}
        if qc.get("quant_method") == "fp8":
            c.quantization = "fp8_block"
        elif qc.get("quant_method") in ("ascend_compressed_tensors", "compressed-tensors", "compressed_tensors"):
            c.quantization = "w8a8_int8"
        return c

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        return cls.from_hf_dict(json.loads((Path(path) / "config.json").read_text()))


# ------------------------------------------------------------------------------------------------
# Named configurations
# ------------------------------------------------------------------------------------------------
def tiny_deepseek_v3(**kw) -> ModelConfig:
    """CPU mock: 2 layers (dense, then MoE), hidden 256, 4 heads, q_lora 128, kv_lora 64, nope 32,
    rope 16, v 32, 8 routed experts (inter 128) top-2 softmax + 1 shared, vocab 1024."""
    c = ModelConfig(architecture="DeepseekV3ForCausalLM", name="tiny-deepseek-v3", vocab_size=1024, hidden_size=256,
                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, q_lora_rank=128,
                    kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, intermediate_size=512,
                    moe_intermediate_size=128, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
                    first_k_dense_replace=1, scoring_func="softmax", topk_method="greedy", norm_topk_prob=False,
                    dtype="float32", max_position_embeddings=512)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def small_deepseek_gpu(**kw) -> ModelConfig:
    """Small MLA+MoE model with the kernel-native head shapes (kv_lora 512, rope 64, nope 128, v 128)."""
    c = ModelConfig(architecture="DeepseekV3ForCausalLM", name="small-deepseek", vocab_size=4096, hidden_size=1024,
                    num_hidden_layers=3, num_attention_heads=16, num_key_value_heads=16, q_lora_rank=512,
                    kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                    intermediate_size=2048, moe_intermediate_size=512, n_routed_experts=16, n_shared_experts=1,
                    num_experts_per_tok=4, first_k_dense_replace=1, scoring_func="sigmoid", topk_method="noaux_tc",
                    n_group=4, topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.5,
                    max_position_embeddings=4096)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def deepseek_v2_lite(**kw) -> ModelConfig:
    c = ModelConfig(architecture="DeepseekV2ForCausalLM", name="deepseek-v2-lite", vocab_size=102400,
                    hidden_size=2048, num_hidden_layers=27, num_attention_heads=16, num_key_value_heads=16,
                    q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                    intermediate_size=10944, moe_intermediate_size=1408, n_routed_experts=64, n_shared_experts=2,
                    num_experts_per_tok=6, first_k_dense_replace=1, scoring_func="softmax", topk_method="greedy",
                    n_group=1, topk_group=1, norm_topk_prob=False, routed_scaling_factor=1.0, rope_theta=10000.0,
                    rope_scaling={"type": "yarn", "factor": 40, "original_max_position_embeddings": 4096,
                                  "beta_fast": 32, "beta_slow": 1, "mscale": 0.707, "mscale_all_dim": 0.707},
                    max_position_embeddings=163840)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def deepseek_v3(**kw) -> ModelConfig:
    c = ModelConfig(architecture="DeepseekV3ForCausalLM", name="deepseek-v3-671b", vocab_size=129280,
                    hidden_size=7168, num_hidden_layers=61, num_attention_heads=128, num_key_value_heads=128,
                    q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                    intermediate_size=18432, moe_intermediate_size=2048, n_routed_experts=256, n_shared_experts=1,
                    num_experts_per_tok=8, first_k_dense_replace=3, scoring_func="sigmoid", topk_method="noaux_tc",
                    n_group=8, topk_group=4, norm_topk_prob=True, routed_scaling_factor=2.5, rope_theta=10000.0,
                    rope_scaling={"type": "yarn", "factor": 40, "original_max_position_embeddings": 4096,
                                  "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0},
                    max_position_embeddings=163840, num_nextn_predict_layers=1, quantization="fp8_block")
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def qwen3_30b_a3b(**kw) -> ModelConfig:
    c = ModelConfig(architecture="Qwen3MoeForCausalLM", name="qwen3-30b-a3b", vocab_size=151936, hidden_size=2048,
                    num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128, use_mla=False,
                    intermediate_size=6144, moe_intermediate_size=768, n_routed_experts=128, n_shared_experts=0,
                    num_experts_per_tok=8, first_k_dense_replace=0, scoring_func="softmax", topk_method="greedy",
                    norm_topk_prob=True, rope_theta=1e6, qk_norm=True, max_position_embeddings=40960)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def qwen2_small(**kw) -> ModelConfig:
    c = ModelConfig(architecture="Qwen2ForCausalLM", name="qwen2-small", vocab_size=4096, hidden_size=1024,
                    num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128, use_mla=False,
                    intermediate_size=2816, n_routed_experts=0, attention_bias=True, rope_theta=1e6,
                    max_position_embeddings=4096)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def tiny_qwen3_moe(**kw) -> ModelConfig:
    """CPU-sized GQA MoE in the shape of Qwen3-MoE: 2 layers, 4 q / 2 kv heads of 32 dims with q/k norm, 8 experts
    top-2 with renormalised softmax routing, no shared expert."""
    c = ModelConfig(architecture="Qwen3MoeForCausalLM", name="tiny-qwen3-moe", vocab_size=1024, hidden_size=128,
                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32, use_mla=False,
                    intermediate_size=256, moe_intermediate_size=64, n_routed_experts=8, n_shared_experts=0,
                    num_experts_per_tok=2, first_k_dense_replace=0, scoring_func="softmax", topk_method="greedy",
                    norm_topk_prob=True, rope_theta=1e6, qk_norm=True, dtype="float32", max_position_embeddings=512)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


PRESETS = {
    "tiny-deepseek-v3": tiny_deepseek_v3,
    "tiny-qwen3-moe": tiny_qwen3_moe,
    "small-deepseek": small_deepseek_gpu,
    "deepseek-v2-lite": deepseek_v2_lite,
    "deepseek-v3": deepseek_v3,
    "qwen3-30b-a3b": qwen3_30b_a3b,
    "qwen2-small": qwen2_small,
}


def get_config(name_or_path: str, **kw) -> ModelConfig:
    if name_or_path in PRESETS:
        return PRESETS[name_or_path](**kw)
    c = ModelConfig.from_pretrained(name_or_path)
    for k, v in kw.items():
        setattr(c, k, v)
    return c
