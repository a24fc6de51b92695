"""Platform plugin (reference: omni/adaptors/vllm/platform.py:131-463).

``register()`` is the ``vllm.platform_plugins`` entry point and returns the platform class path.  The platform
object carries what the host engine asks a platform: device naming, the worker class, block size, attention
backend choice by model type, memory info, and ``check_and_update_config`` which turns the additional-config
JSON into runner settings (gears -> CUDA-graph buckets, hybrid scheduler, async scheduling, Omni-Attention).
When no compatible host engine is installed the same object configures the in-repo engine."""
from __future__ import annotations

import logging
from typing import Optional

import torch

from ...config import AdditionalConfig, load_model_extra_config

logger = logging.getLogger("omni_infer_b200.platform")

PLATFORM_CLS = "omni_infer_b200.adaptors.vllm.platform.B200Platform"
WORKER_CLS = "omni_infer_b200.adaptors.vllm.worker.B200Worker"


def register() -> Optional[str]:
    """Entry point ``vllm.platform_plugins``: returns the platform class path, or None without a CUDA device
    unless the no-GPU mock is requested."""
    import os

    if torch.cuda.is_available() or os.environ.get("NO_GPU_MOCK", os.environ.get("NO_NPU_MOCK", "0")) == "1":
        return PLATFORM_CLS
    return None


def ensure_v1_engine() -> None:
    """The reference forces the host engine's V1 architecture; the in-repo engine is built that way."""


class ConfigUpdater:
    @staticmethod
    def update_engine_config(engine_cfg, additional_config=None, model_extra_cfg_path: Optional[str] = None):
        """Apply additional-config + extra-config to an :class:`EngineConfig` in place and return it."""
        add = AdditionalConfig.from_json(additional_config or {})
        extra = load_model_extra_config(model_extra_cfg_path, add.__dict__ if False else None)
        g = add.graph_model_compile_config
        engine_cfg.enforce_eager = not g.use_cuda_graph
        engine_cfg.decode_gear_list = g.update_gear_options(engine_cfg.max_num_seqs, engine_cfg.num_speculative_tokens)
        engine_cfg.async_schedule = bool(add.async_schedule)
        engine_cfg.num_step = max(1, add.multi_step)
        engine_cfg.block_size = engine_cfg.block_size or 128
        engine_cfg.enable_omni_attn = bool(add.enable_omni_attn)
        engine_cfg.omni_attn_config = add.omni_attn_config
        if add.async_pull_kv and engine_cfg.kv_transfer_config is not None:
            engine_cfg.kv_transfer_config = dict(engine_cfg.kv_transfer_config, async_pull_kv=True)
        oc = extra.operator_opt_config
        if oc.decode_gear_list:
            engine_cfg.decode_gear_list = list(oc.decode_gear_list)
        if oc.use_omni_placement and oc.omni_placement_config_path:
            engine_cfg.placement_config = {"config_path": oc.omni_placement_config_path}
        engine_cfg.ep_backend = "fused" if oc.moe_dispatch_combine else "nccl"
        engine_cfg.tp_size = max(1, engine_cfg.tp_size)
        return engine_cfg


class B200Platform:
    _enum = "OOT"
    device_name = "cuda"
    device_type = "cuda"
    dispatch_key = "CUDA"
    ray_device_key = "GPU"
    device_control_env_var = "CUDA_VISIBLE_DEVICES"
    supported_quantization = ["fp8", "fp8_block", "ascend_compressed_tensors", "compressed-tensors"]
    simple_compile_backend = "eager"

    @classmethod
    def pre_register_and_update(cls, parser=None) -> None:
        from ...models import register_model
        from ...quantization import config as _q  # noqa: F401  (registers the quantization config names)

        register_model()

    @classmethod
    def check_and_update_config(cls, engine_cfg, additional_config=None) -> None:
        ConfigUpdater.update_engine_config(engine_cfg, additional_config)

    @classmethod
    def get_attn_backend_cls(cls, use_mla: bool) -> str:
        return ("omni_infer_b200.layers.mla.MLAAttention" if use_mla else "omni_infer_b200.layers.gqa.GQAAttention")

    @classmethod
    def get_device_communicator_cls(cls) -> str:
        return "omni_infer_b200.parallel.parallel_state.GroupCoordinator"

    @classmethod
    def get_worker_cls(cls) -> str:
        return WORKER_CLS

    @classmethod
    def mem_get_info(cls, device=None):
        if torch.cuda.is_available():
            return torch.cuda.mem_get_info(device)
        import psutil
        vm = psutil.virtual_memory()
        return vm.available, vm.total

    @classmethod
    def is_pin_memory_available(cls) -> bool:
        import os
        return torch.cuda.is_available() and os.environ.get("NO_GPU_MOCK", "0") != "1"

    @classmethod
    def get_device_name(cls, device_id: int = 0) -> str:
        return torch.cuda.get_device_name(device_id) if torch.cuda.is_available() else "cpu"

    @classmethod
    def synchronize(cls) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @classmethod
    def use_all_gather(cls) -> bool:
        return True
