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
        pc = extra.parall_config
        engine_cfg.dense_mlp_tp_size = max(1, int(pc.dense_mlp_tp_size))
        engine_cfg.o_proj_tp_size = max(1, int(pc.o_proj_tp_size))
        engine_cfg.shared_expert_ranks = max(0, int(pc.redundancy_shared_expert_num))
        return engine_cfg


def _host_platform_base():
    """The host engine's ``Platform`` base class and its out-of-tree enum value when that engine imports; a plain
    ``object`` otherwise, so that the in-repo engine does not depend on it."""
    try:
        from vllm.platforms.interface import Platform, PlatformEnum
        return Platform, PlatformEnum.OOT
    except Exception:  # noqa: BLE001  (absent, or built for another torch)
        return object, "OOT"


_Base, _OOT = _host_platform_base()


class B200Platform(_Base):
    _enum = _OOT
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
        """Called by the host engine with its ``VllmConfig`` (worker class, block size 128, additional-config
        switches; reference: platform.py:179-259, 375-390) or by the in-repo engine with an ``EngineConfig``."""
        if hasattr(engine_cfg, "parallel_config"):
            pc = engine_cfg.parallel_config
            if getattr(pc, "worker_cls", "auto") in ("auto", None):
                pc.worker_cls = WORKER_CLS
            cc = getattr(engine_cfg, "cache_config", None)
            if cc is not None and not getattr(cc, "block_size", None):
                cc.block_size = 128
            add = getattr(engine_cfg, "additional_config", None) or {}
            sc = getattr(engine_cfg, "scheduler_config", None)
            if sc is not None and isinstance(add, dict) and add.get("enable_hybrid_graph_mode"):
                sc.scheduler_cls = "omni_infer_b200.engine.scheduler.Scheduler"
            return
        ConfigUpdater.update_engine_config(engine_cfg, additional_config)

    @classmethod
    def get_attn_backend_cls(cls, use_mla=False, *args, **kwargs) -> str:
        # the host engine passes (selected_backend, attn_selector_config, ...); MLA models are told apart by use_mla
        if not isinstance(use_mla, bool):
            sel = args[0] if args else kwargs.get("attn_selector_config")
            use_mla = bool(getattr(sel, "use_mla", kwargs.get("use_mla", False)))
        return ("omni_infer_b200.layers.mla.MLAAttention" if use_mla else "omni_infer_b200.layers.gqa.GQAAttention")

    @classmethod
    def get_device_capability(cls, device_id: int = 0):
        if not torch.cuda.is_available():
            return None
        major, minor = torch.cuda.get_device_capability(device_id)
        try:
            from vllm.platforms.interface import DeviceCapability
            return DeviceCapability(major=major, minor=minor)
        except Exception:  # noqa: BLE001
            return (major, minor)

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        return torch.cuda.get_device_properties(device_id).total_memory if torch.cuda.is_available() else 0

    @classmethod
    def set_device(cls, device) -> None:
        if torch.cuda.is_available():
            torch.cuda.set_device(device)

    @classmethod
    def get_current_memory_usage(cls, device=None) -> float:
        if not torch.cuda.is_available():
            return 0.0
        torch.cuda.reset_peak_memory_stats(device)
        return float(torch.cuda.max_memory_allocated(device))

    @classmethod
    def inference_mode(cls):
        return torch.inference_mode(mode=True)

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
