"""Quantization configuration (reference: omni/quantization/compressed_tensors/compressed_tensors.py:40-262).

Recognised formats:
  * ``fp8`` / HF DeepSeek-V3: e4m3 weights + ``weight_scale_inv`` per 128x128 block, dynamic 1x128 activations
  * ``ascend_compressed_tensors`` / ``compressed-tensors`` int8 w8a8 dynamic per token (the reference's native
    layout, described by ``quant_model_description.json``): loaded, de-quantised and re-quantised to block e4m3
  * w4a8 is detected and rejected (the reference only carries stubs for it)
``get_quant_method(layer_kind, prefix)`` mirrors the reference's dispatch: Linear / FusedMoE / attention KV."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

QUANT_NAMES = ("ascend_compressed_tensors", "compressed-tensors", "compressed_tensors", "fp8")


@dataclass
class QuantConfig:
    name: str = "none"                       # none | fp8_block | w8a8_int8
    ignore: list = field(default_factory=list)
    weight_block_size: tuple = (128, 128)
    kv_cache_scheme: Optional[str] = None    # fa_quant_type of the reference (int8 KV) - accepted, stored as bf16
    description: dict = field(default_factory=dict)

    @classmethod
    def from_hf_config(cls, hf: dict, model_dir: Optional[str] = None) -> "QuantConfig":
        qc = hf.get("quantization_config") or {}
        method = qc.get("quant_method", "")
        c = cls()
        if method == "fp8":
            c.name = "fp8_block"
            c.weight_block_size = tuple(qc.get("weight_block_size", (128, 128)))
        elif method in QUANT_NAMES:
            c.name = "w8a8_int8"
            c.ignore = list(qc.get("ignore", []))
            groups = qc.get("config_groups", {})
            for g in groups.values():
                w = g.get("weights", {})
                nb = w.get("num_bits")
                nb = nb.get("weight", 8) if isinstance(nb, dict) else nb     # lenient form used by the reference
                if nb == 4:
                    raise NotImplementedError("w4a8 checkpoints are not supported (the reference ships stubs only)")
            c.kv_cache_scheme = qc.get("kv_cache_scheme") or qc.get("fa_quant_type")
        if model_dir:
            p = Path(model_dir) / "quant_model_description.json"
            if p.exists():
                c.description = json.loads(p.read_text())
                if c.name == "none":
                    c.name = "w8a8_int8"
        return c

    def is_ignored(self, prefix: str) -> bool:
        if any(prefix == i or prefix.endswith(i) or i in prefix for i in self.ignore):
            return True
        d = self.description.get(prefix + ".weight")
        return d is not None and str(d).upper() in ("FLOAT", "BF16", "FP16")

    def get_quant_method(self, layer_kind: str, prefix: str) -> str:
        """'none' | 'fp8_block' for a layer of kind 'linear' | 'moe' | 'attention'."""
        if self.name == "none" or self.is_ignored(prefix):
            return "none"
        if layer_kind == "attention":
            return "none"          # KV cache stays bf16
        return "fp8_block"         # int8 checkpoints are re-quantised to block e4m3 at load


def override_quantization_method(hf_quant_cfg: dict, user_quant: Optional[str]) -> Optional[str]:
    """Same hook as the reference: claim checkpoints produced for it."""
    if hf_quant_cfg and hf_quant_cfg.get("quant_method") in QUANT_NAMES[:3]:
        return "ascend_compressed_tensors"
    return None
