"""B200-native MoE inference accelerator.

Sub-packages: ``ops`` (sm_100a kernels and their fp32 PyTorch references), ``layers`` and
``models`` (DeepSeek-V2/V3 MLA+MoE, MTP, Qwen GQA/MoE), ``parallel`` (process groups, symmetric
heap, fused collectives), ``engine`` (scheduler / KV manager / engine core / API server),
``adaptors`` (platform, worker, model runner), ``quantization``, ``accelerators`` (PD
disaggregation, Omni-Attention KV compression, OmniPlacement, global proxy launcher), ``cli``.
"""
__version__ = "0.2.0"
