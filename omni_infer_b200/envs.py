"""Lazy environment-variable registry (reference: omni/adaptors/vllm/envs.py:29-64).

``envs.NAME`` evaluates the variable on every access, so tests can change the environment at run time.
Ascend-only switches of the reference are accepted and ignored (listed in ``IGNORED``) so that existing
launch scripts keep working."""
from __future__ import annotations

import os
from typing import Any, Callable

_B = lambda name, default="0": (lambda: os.environ.get(name, default) == "1")  # noqa: E731
_I = lambda name, default: (lambda: int(os.environ.get(name, default)))        # noqa: E731
_S = lambda name, default=None: (lambda: os.environ.get(name, default))        # noqa: E731

env_variables: dict[str, Callable[[], Any]] = {
    # engine / platform
    "OMNI_USE_FUSED_EP": _B("OMNI_USE_FUSED_EP", "1"),          # role of VLLM_ENABLE_MC2
    "OMNI_EP_WAIT_MS": _I("OMNI_EP_WAIT_MS", "2000"),
    "MODEL_EXTRA_CFG_PATH": _S("MODEL_EXTRA_CFG_PATH", ""),
    "OMNI_GRAPH_CACHE_HOME": _S("OMNI_GRAPH_CACHE_HOME", os.path.expanduser("~/.cache/omni_infer_b200")),
    "NO_GPU_MOCK": _B("NO_GPU_MOCK"),
    "OMNI_INIT_ON_HOST": _B("OMNI_INIT_ON_HOST"),               # random-init weights drawn on the CPU (tiny models)
    "FORCE_ENABLE_CHUNK_PREFILL": _B("FORCE_ENABLE_CHUNK_PREFILL"),
    # PD disaggregation
    "ROLE": _S("ROLE", "mixed"),
    "PREFILL_POD_NUM": _I("PREFILL_POD_NUM", "1"),
    "DECODE_POD_NUM": _I("DECODE_POD_NUM", "1"),
    "OMNI_KV_CONTROL_PORT": _I("OMNI_KV_CONTROL_PORT", "5568"),
    "OMNI_KV_SYNC_TIMEOUT_MS": _I("OMNI_KV_SYNC_TIMEOUT_MS", "20000"),
    "OMNI_KV_RETRY": _I("OMNI_KV_RETRY", "3"),
    "OMNI_KV_RETRY_WAIT_S": _I("OMNI_KV_RETRY_WAIT_S", "2"),
    "GLOBAL_TOPOLOGY": _S("GLOBAL_TOPOLOGY", ""),
    # serving front end
    "TOKENIZER_PROC_POOL": _B("TOKENIZER_PROC_POOL"),
    "TOKENIZER_WORKER_NUM": _I("TOKENIZER_WORKER_NUM", "4"),
    "TOKENIZER_PROC_POOL_THRES": _I("TOKENIZER_PROC_POOL_THRES", "2048"),
    "TOKENIZER_AFFINITY_CORES": _S("TOKENIZER_AFFINITY_CORES", ""),
    "OMNI_REUSE_PREFILLED_TOKENS": _B("OMNI_REUSE_PREFILLED_TOKENS", "1"),
    "OMNI_SKIP_DECODE_TOKENIZE": _B("OMNI_SKIP_DECODE_TOKENIZE", "1"),
    # mock model / profiling
    "RANDOM_MODE": _B("RANDOM_MODE"),
    "CAPTURE_MODE": _B("CAPTURE_MODE"),
    "REPLAY_MODE": _B("REPLAY_MODE"),
    "KV_CACHE_MODE": _B("KV_CACHE_MODE"),
    "PREFILL_PROCESS": _B("PREFILL_PROCESS"),
    "FORWARD_TIME": _I("FORWARD_TIME", "0"),
    "SIMULATE_ELAPSED_TIME": _B("SIMULATE_ELAPSED_TIME"),
    "MOCK_CAPTURE_DIR": _S("MOCK_CAPTURE_DIR", "/tmp/omni_mock"),
    "MOCK_CAPTURE_FILE": _S("MOCK_CAPTURE_FILE", "capture.jsonl"),
    "MOCK_COMPUTE_LOGITS": _B("MOCK_COMPUTE_LOGITS"),
    "PROFILING_NAMELIST": _S("PROFILING_NAMELIST", ""),
    "PROFILING_FORWARD": _B("PROFILING_FORWARD"),
    "VLLM_TORCH_PROFILER_DIR": _S("VLLM_TORCH_PROFILER_DIR", "./profiler_traces"),
}

IGNORED = ("ASCEND_PLATFORM", "USING_LCCL_COM", "HCCL_CONNECT_TIMEOUT", "HCCL_EXEC_TIMEOUT", "TORCHAIR_CACHE_HOME",
           "PROMPT_DEVICE_ID", "DECODE_DEVICE_ID", "ASCEND_RT_VISIBLE_DEVICES", "CPU_AFFINITY_CONF")


def __getattr__(name: str):
    if name in env_variables:
        return env_variables[name]()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return list(env_variables.keys())
