"""One worker process per GPU (reference: NPUWorker, omni/adaptors/vllm/worker/npu_worker.py:68-344):
device selection with data-parallel local-rank math, NCCL + gloo initialisation, model load, memory
profiling and KV sizing with a host-side agreement across ranks, CUDA-graph warm-up, step execution,
dummy batches for idle data-parallel ranks, and the torch profiler toggle."""
from __future__ import annotations

import logging
import os
from typing import Optional

import torch
import torch.distributed as dist

from ...models.config import ModelConfig
from ...parallel import get_parallel_state, init_distributed
from .model_runner import ModelRunner, RunnerConfig

logger = logging.getLogger("omni_infer_b200.worker")


class B200Worker:
    def __init__(self, model_cfg: ModelConfig, runner_cfg: RunnerConfig, *, tp_size: int = 1, device: Optional[str] = None,
                 planner=None, kv_connector=None, dense_mlp_tp_size: int = 1, o_proj_tp_size: int = 1, pp_size: int = 1):
        self.model_cfg, self.runner_cfg = model_cfg, runner_cfg
        self.tp_size, self.dense_mlp_tp_size, self.o_proj_tp_size = tp_size, dense_mlp_tp_size, o_proj_tp_size
        self.pp_size = pp_size
        self.requested_device = device
        self.planner, self.kv_connector = planner, kv_connector
        self.runner: Optional[ModelRunner] = None
        self.profiler = None
        self.device = None

    # ------------------------------------------------------------------ bring-up
    def init_device(self) -> None:
        no_gpu = os.environ.get("NO_GPU_MOCK", os.environ.get("NO_NPU_MOCK", "0")) == "1"
        use_cuda = torch.cuda.is_available() and not no_gpu and self.requested_device != "cpu"
        ps = init_distributed(backend="nccl" if use_cuda else "gloo", tp_size=self.tp_size,
                              dense_mlp_tp_size=self.dense_mlp_tp_size, o_proj_tp_size=self.o_proj_tp_size,
                              pp_size=self.pp_size) \
            if int(os.environ.get("WORLD_SIZE", "1")) > 1 else get_parallel_state()
        if use_cuda:
            # with one engine per data-parallel rank, LOCAL_RANK already accounts for the DP offset
            self.device = torch.device("cuda", ps.local_rank if ps.world_size > 1 else torch.cuda.current_device())
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        if ps.world_size > 1 and not self.runner_cfg.attn_tp:
            self.model_cfg.dense_mlp_tp_size = max(1, min(self.dense_mlp_tp_size, ps.world_size))
            self.model_cfg.o_proj_tp_size = max(1, min(self.o_proj_tp_size, ps.world_size))
        self.runner = ModelRunner(self.model_cfg, self.runner_cfg, self.device, planner=self.planner,
                                  kv_connector=self.kv_connector)

    def load_model(self, weights=None, seed: Optional[int] = 0) -> None:
        self.runner.load_model(weights, seed)

    def determine_available_memory(self) -> int:
        """Profile one worst-case prefill, size the KV cache from what is left, and agree on the minimum
        block count over all ranks on the CPU group (omni/adaptors/vllm/worker/npu_worker.py:166-214)."""
        r = self.runner
        if self.device.type == "cuda" and not r.cfg.num_kv_blocks:
            torch.cuda.reset_peak_memory_stats(self.device)
            try:
                r.profile_run()
            finally:
                torch.cuda.empty_cache()
        n = r.determine_num_blocks()
        ps = get_parallel_state()
        if ps.world_size > 1:
            t = torch.tensor([n], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=ps.group("cpu").group)
            n = int(t.item())
        return n

    def initialize_cache(self, num_blocks: int) -> None:
        self.runner.initialize_kv_cache(num_blocks)

    def compile_or_warm_up_model(self) -> None:
        self.runner.capture_model()

    # ------------------------------------------------------------------ stepping
    def execute_model(self, scheduler_output):
        return self.runner.execute_model(scheduler_output)

    def execute_dummy_batch(self) -> None:
        self.runner.execute_dummy_batch()

    # ------------------------------------------------------------------ profiling (start_profile / stop_profile)
    def profile(self, is_start: bool = True) -> None:
        if is_start:
            d = os.environ.get("VLLM_TORCH_PROFILER_DIR", "./profiler_traces")
            acts = [torch.profiler.ProfilerActivity.CPU]
            if self.device.type == "cuda":
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.profiler = torch.profiler.profile(activities=acts,
                                                   on_trace_ready=torch.profiler.tensorboard_trace_handler(d))
            self.profiler.start()
        elif self.profiler is not None:
            self.profiler.stop()
            self.profiler = None

    # sleep / wake are accepted for interface parity; weights stay resident
    def sleep(self, level: int = 1) -> None:
        logger.warning("sleep mode is not supported; ignoring")

    def wake_up(self) -> None:
        logger.warning("sleep mode is not supported; ignoring")
