"""Typed configuration loadable from the reference's three sources: the ``--additional-config`` JSON, the
``MODEL_EXTRA_CFG_PATH`` JSON file, and environment variables (omni/models/common/config/model_config.py:10-131,
omni/adaptors/vllm/platform.py:179-259, omni/adaptors/vllm/compilation/compile_config.py:68-111).

Key names are kept where the feature exists here; keys that only make sense on the reference's hardware are
accepted and ignored with a warning, so existing config files load unchanged."""
from __future__ import annotations

import json
import logging
import os
from dataclasses import dataclass, field, fields
from typing import Any, Optional

logger = logging.getLogger("omni_infer_b200.config")


@dataclass
class ModelParallelConfig:
    dense_mlp_tp_size: int = 1
    dp_size: int = 1
    o_proj_tp_size: int = 1
    redundancy_shared_expert_num: int = 0


@dataclass
class ModelOperatorOptConfig:
    enable_kv_rmsnorm_rope_cache: bool = True     # always fused here (norm_rope.cu)
    prefill_dispatch_combine: bool = False        # prefill uses the all-to-all path
    enable_node_mlp: bool = False
    moe_multi_stream_tune: bool = True            # shared expert on a side stream
    best_ep: bool = False                         # forced-balance routing (benchmark aid)
    merge_qkv: bool = True                        # q_a + kv_a merged projection
    two_stage_comm: bool = False
    use_chunked_prefill: bool = False
    use_w8a8_dynamic_quant: bool = True
    gmm_nz: bool = False
    moe_dispatch_combine: bool = True             # fused NVLink dispatch/combine on decode
    use_omni_placement: bool = False
    omni_placement_config_path: Optional[str] = None
    enable_fusion_spec: bool = False
    enable_alltoall: bool = False
    enable_pd_separated: bool = False
    use_super_kernel: bool = False
    use_mlaprolog: bool = False
    opt_w2_scale_cast: bool = False
    enable_mc2_v2: bool = False
    decode_gear_list: list = field(default_factory=lambda: [])
    control_accept_rate: float = -1.0
    enable_prefill_micro_batch: bool = False
    use_prefetch: bool = False
    expert_gate_up_prefetch: int = 0
    expert_down_prefetch: int = 0
    attn_prefetch: int = 0
    fa_quantization: bool = False


_ASCEND_ONLY = {"gmm_nz", "use_super_kernel", "use_mlaprolog", "opt_w2_scale_cast", "enable_mc2_v2", "two_stage_comm",
                "use_prefetch", "expert_gate_up_prefetch", "expert_down_prefetch", "attn_prefetch", "enable_node_mlp"}


@dataclass
class ModelExtraConfig:
    parall_config: ModelParallelConfig = field(default_factory=ModelParallelConfig)
    operator_opt_config: ModelOperatorOptConfig = field(default_factory=ModelOperatorOptConfig)


def _fill(dc, data: dict, where: str) -> None:
    known = {f.name for f in fields(dc)}
    for k, v in (data or {}).items():
        if k in known:
            setattr(dc, k, v)
            if k in _ASCEND_ONLY and v:
                logger.warning("%s.%s is specific to the reference hardware and has no effect here", where, k)
        else:
            logger.warning("unknown key %s.%s ignored", where, k)


def load_model_extra_config(path: Optional[str] = None, additional_config: Optional[dict] = None) -> ModelExtraConfig:
    """File given by ``path`` or ``MODEL_EXTRA_CFG_PATH``; ``additional_config`` overrides it."""
    cfg = ModelExtraConfig()
    path = path or os.environ.get("MODEL_EXTRA_CFG_PATH", "")
    if path:
        data = json.loads(open(path).read())
        _fill(cfg.parall_config, data.get("model_parallel_config", {}), "model_parallel_config")
        _fill(cfg.operator_opt_config, data.get("operator_optimizition_config",
                                                data.get("operator_optimization_config", {})), "operator_opt_config")
    if additional_config:
        _fill(cfg.parall_config, additional_config.get("model_parallel_config", {}), "additional.model_parallel_config")
        _fill(cfg.operator_opt_config, additional_config.get("operator_optimizition_config", {}), "additional.operator_opt_config")
    return cfg


@dataclass
class GraphCompileConfig:
    """``graph_model_compile_config`` of the additional config: gears become CUDA-graph buckets."""
    level: int = 1
    use_cuda_graph: bool = True
    decode_gear_list: list = field(default_factory=list)
    block_num_floating_range: int = 30

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> "GraphCompileConfig":
        c = cls()
        d = d or {}
        c.level = int(d.get("level", 1))
        c.use_cuda_graph = c.level > 0 and not d.get("enforce_eager", False)
        c.decode_gear_list = list(d.get("decode_gear_list", []))
        for k in ("use_aclgraph", "use_ge_graph_cached", "backend"):
            if k in d:
                logger.warning("graph_model_compile_config.%s is specific to the reference's graph compiler; ignored", k)
        return c

    def update_gear_options(self, max_num_seqs: int, num_speculative_tokens: int) -> list:
        """Default gear = max_num_seqs * (1 + speculative tokens) token rows, i.e. the full batch bucket."""
        if not self.decode_gear_list:
            self.decode_gear_list = [max_num_seqs]
        return self.decode_gear_list


@dataclass
class AdditionalConfig:
    graph_model_compile_config: GraphCompileConfig = field(default_factory=GraphCompileConfig)
    enable_hybrid_graph_mode: bool = True
    async_schedule: bool = False
    multi_step: int = 1
    async_pull_kv: bool = False
    enable_omni_attn: bool = False
    omni_attn_config: Optional[dict] = None

    @classmethod
    def from_json(cls, text_or_dict: Any) -> "AdditionalConfig":
        d = json.loads(text_or_dict) if isinstance(text_or_dict, str) else dict(text_or_dict or {})
        c = cls()
        c.graph_model_compile_config = GraphCompileConfig.from_dict(d.get("graph_model_compile_config"))
        for k in ("enable_hybrid_graph_mode", "async_schedule", "async_pull_kv", "enable_omni_attn", "omni_attn_config"):
            if k in d:
                setattr(c, k, d[k])
        ms = d.get("multi_step", 1)
        c.multi_step = int(ms) if not isinstance(ms, bool) else (2 if ms else 1)
        return c
