"""Device ops.  Every function takes tensors; CUDA tensors run the hand-written sm_100a kernels from
``csrc/kernels`` (through ``libomni_kernels.so``), CPU tensors run the fp32 PyTorch reference of the
same op, which is also the oracle in the tests."""
from . import _native  # noqa: F401
from . import attention  # noqa: F401
from .attention import attn_prefill_ref, gqa_decode_ref, mla_decode, mla_decode_ref  # noqa: F401
from .basic import (embedding, mla_kv_rope_cache, quant_fp8_block, rmsnorm, rope_cos_sin_table,  # noqa: F401
                    rope_interleaved_ref, rope_neox_ref, rope_qk_cache, silu_mul)
from .gemm import (FP8, bmm_heads, dequant_act_ref, dequant_weight_ref, gemm, gemm_ref, quant_fp8_block_ref,  # noqa: F401
                   quant_weight_fp8_block_ref)
from .moe import MoePermutation, moe_combine, moe_permute, router_topk, router_topk_ref  # noqa: F401
from .sampling import apply_penalties, apply_penalties_ref, argmax, mtp_verify, omni_attn_slots, sample_topk_topp, step_advance  # noqa: F401
