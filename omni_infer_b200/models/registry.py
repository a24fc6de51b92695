"""Model registry: architecture name -> class, mirroring ``register_model()`` of the reference
(omni/models/__init__.py:14-60), including the mock wrappers selected by environment variables."""
from __future__ import annotations

import os

_REGISTRY: dict = {}


def register(name: str, target) -> None:
    _REGISTRY[name] = target


def _lazy():
    if _REGISTRY:
        return
    from .deepseek import DeepseekV2ForCausalLM, DeepseekV3ForCausalLM
    from .deepseek_mtp import DeepSeekMTPModel, DeepSeekMTPModelDuo, DeepSeekMTPModelTres
    from .qwen import Qwen2ForCausalLM, Qwen3MoeForCausalLM

    table = {
        "DeepseekV2ForCausalLM": DeepseekV2ForCausalLM,
        "DeepseekV3ForCausalLM": DeepseekV3ForCausalLM,
        "DeepSeekMTPModel": DeepSeekMTPModel,
        "DeepSeekMTPModelDuo": DeepSeekMTPModelDuo,
        "DeepSeekMTPModelTres": DeepSeekMTPModelTres,
        "Qwen2ForCausalLM": Qwen2ForCausalLM,
        "Qwen3MoeForCausalLM": Qwen3MoeForCausalLM,
    }
    if any(os.environ.get(k) == "1" for k in ("RANDOM_MODE", "CAPTURE_MODE", "REPLAY_MODE")):
        from .mock import mock_model_class_factory
        for k in ("DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM", "Qwen2ForCausalLM", "Qwen3MoeForCausalLM"):
            table[k] = mock_model_class_factory(table[k])
    _REGISTRY.update(table)


def register_model() -> dict:
    """Entry point name kept from the reference's ``vllm.general_plugins`` hook."""
    _lazy()
    try:      # the response parsers of the Pangu models, under the name "pangu" in the host engine's parser managers
        from .pangu.host_engine import register_with_host_engine
        register_with_host_engine()
        from ..quantization.host_engine import register_with_host_engine as register_quantization
        register_quantization()
    except Exception:  # noqa: BLE001  (no host engine: the in-repo API server has its own wiring)
        pass
    try:      # architecture names -> these classes in the host engine's model registry (lazy form: nothing is imported)
        from vllm import ModelRegistry
        for arch, cls in _REGISTRY.items():
            ModelRegistry.register_model(arch, f"{cls.__module__}:{cls.__qualname__}")
    except Exception:  # noqa: BLE001
        pass
    if os.environ.get("PROFILING_NAMELIST"):
        from ..utils.profiler_patches import apply_patches
        apply_patches(os.environ["PROFILING_NAMELIST"])
    return dict(_REGISTRY)


def get_model_class(architecture: str):
    _lazy()
    if architecture not in _REGISTRY:
        raise KeyError(f"unknown architecture {architecture!r}; known: {sorted(_REGISTRY)}")
    return _REGISTRY[architecture]


def build_model(cfg, device=None, planner=None, seed=None):
    cls = get_model_class(cfg.architecture)
    model = cls(cfg, device=device, planner=planner)
    if seed is not None:
        from ..quantization.loader import init_random_weights
        init_random_weights(model, seed)
    return model
