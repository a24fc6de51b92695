"""The quantisation format names of this package in the host engine's registry, so that its configuration layer
accepts ``--quantization ascend_compressed_tensors`` (the name the reference registers,
omni/quantization/compressed_tensors/compressed_tensors.py:40) for a checkpoint that this package's own worker then
loads (quantization/loader.py).  The adapter describes the format; it creates no layers of the host engine."""
from __future__ import annotations

from .config import QuantConfig

NAME = "ascend_compressed_tensors"


def register_with_host_engine() -> bool:
    try:
        import torch
        from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, register_quantization_config
        from vllm.model_executor.layers.quantization.base_config import QuantizationConfig
    except Exception:  # noqa: BLE001  (no host engine here)
        return False
    if NAME in QUANTIZATION_METHODS:
        return True

    @register_quantization_config(NAME)
    class B200CompressedTensorsConfig(QuantizationConfig):
        """int8 w8a8 compressed-tensors checkpoints (per-channel weight scale / offset, dynamic per-token activations),
        re-quantised to block e4m3 when this package's worker loads them."""

        def __init__(self, inner: QuantConfig = None):
            super().__init__()
            self.inner = inner or QuantConfig(name="w8a8_int8")

        @classmethod
        def get_name(cls) -> str:
            return NAME

        @classmethod
        def get_supported_act_dtypes(cls) -> list:
            return [torch.bfloat16, torch.float16]

        @classmethod
        def get_min_capability(cls) -> int:
            return 100                                  # sm_100

        @staticmethod
        def get_config_filenames() -> list:
            return ["quant_model_description.json"]

        @classmethod
        def from_config(cls, config: dict) -> "B200CompressedTensorsConfig":
            return cls(QuantConfig.from_hf_config({"quantization_config": dict(config, quant_method=config.get("quant_method", NAME))}))

        @classmethod
        def override_quantization_method(cls, hf_quant_cfg, user_quant):
            method = (hf_quant_cfg or {}).get("quant_method", "")
            return NAME if user_quant == NAME or method in (NAME, "compressed-tensors", "compressed_tensors") and user_quant == NAME else None

        def get_quant_method(self, layer, prefix: str):
            return None                                  # the layers are this package's own; nothing to attach here

    return True
