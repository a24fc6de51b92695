"""Building blocks shared by every model: attention metadata, linear layers (bf16 / block-scaled
e4m3), RMSNorm, the SwiGLU MLP."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
from torch import nn

from .. import ops
from ..ops import FP8


@dataclass
class AttnMetadata:
    """Per-step attention inputs built by the model runner.

    The reference carries the same information in AscendMLAMetadata / AscendMetadata
    (omni/models/common/layers/attention/backend/mla.py:105-166): attention state, slot mapping,
    block table, sequence lengths; prefill additionally has ragged query/key offsets."""
    is_prefill: bool
    positions: torch.Tensor                 # [T] int64
    slot_mapping: torch.Tensor              # [T] int64, -1 = do not store
    block_table: torch.Tensor               # [B, max_blocks] int32
    seq_lens: torch.Tensor                  # [B] int32 total kv tokens per request after this step
    # prefill
    cu_q: Optional[torch.Tensor] = None     # [B+1] int32
    cu_k: Optional[torch.Tensor] = None     # [B+1] int32
    query_lens: Optional[list] = None
    context_lens: Optional[list] = None     # cached-prefix tokens per request
    max_q: int = 0
    max_k: int = 0
    kv_gather_slots: Optional[torch.Tensor] = None   # [sum_k] int64 cache slots of the whole context (prefix hits)
    # decode
    tokens_per_req: int = 1                 # 1 + speculative tokens
    q_seq_lens: Optional[torch.Tensor] = None   # [B * tokens_per_req] int32 visible kv tokens per q row
    q_to_seq: Optional[torch.Tensor] = None     # [B * tokens_per_req] int32
    max_seq_len: int = 0
    num_valid: Optional[torch.Tensor] = None    # device int32 scalar: rows beyond are padding
    sample_indices: Optional[torch.Tensor] = None  # rows of hidden states that produce logits
    # Omni-Attention (compressed layers): per-layer-group overrides
    omni: Optional[dict] = None


def _dtype(name: str) -> torch.dtype:
    return {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[name]


class Linear(nn.Module):
    """y = x W^T (+ b).  ``quant='fp8_block'`` stores e4m3 weights with 128x128 scales and quantises the
    activation per (row, 128 columns) unless the caller passes it already quantised."""

    def __init__(self, in_features: int, out_features: int, *, dtype=torch.bfloat16, quant: str = "none",
                 bias: bool = False, device=None):
        super().__init__()
        self.in_features, self.out_features, self.quant = in_features, out_features, quant
        if quant == "fp8_block":
            self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=FP8, device=device),
                                       requires_grad=False)
            self.weight_scale = nn.Parameter(
                torch.ones((out_features + 127) // 128, (in_features + 127) // 128, dtype=torch.float32, device=device),
                requires_grad=False)
        else:
            self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device),
                                       requires_grad=False)
            self.weight_scale = None
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device), requires_grad=False) if bias else None

    def forward(self, x, xq=None, epi: str = "store", out_dtype=None):
        if self.quant == "fp8_block":
            if xq is None:
                xq = ops.quant_fp8_block(x)
            y = ops.gemm(xq[0], self.weight, w_scale=self.weight_scale, x_scale=xq[1], epi=epi, out_dtype=out_dtype)
        else:
            y = ops.gemm(x, self.weight, epi=epi, out_dtype=out_dtype)
        if self.bias is not None:
            y = y + self.bias
        return y


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x, residual=None, quant=False):
        """Returns y, or (y, y_q, scale) with ``quant``; ``residual`` is updated in place to x + residual."""
        return ops.rmsnorm(x, self.weight, self.eps, residual=residual, quant=quant)


class SwiGLUMLP(nn.Module):
    """gate_up (merged, gate rows first) -> SwiGLU fused in the GEMM epilogue -> down."""

    def __init__(self, hidden: int, inter: int, *, dtype=torch.bfloat16, quant="none", device=None):
        super().__init__()
        self.gate_up_proj = Linear(hidden, 2 * inter, dtype=dtype, quant=quant, device=device)
        self.down_proj = Linear(inter, hidden, dtype=dtype, quant=quant, device=device)
        self.quant = quant

    def forward(self, x, xq=None):
        if self.quant == "fp8_block":
            if xq is None:
                xq = ops.quant_fp8_block(x)
            aq = ops.gemm(xq[0], self.gate_up_proj.weight, w_scale=self.gate_up_proj.weight_scale, x_scale=xq[1],
                          epi="swiglu_quant")
            return ops.gemm(aq[0], self.down_proj.weight, w_scale=self.down_proj.weight_scale, x_scale=aq[1])
        act = ops.gemm(x, self.gate_up_proj.weight, epi="swiglu")
        return ops.gemm(act, self.down_proj.weight)
