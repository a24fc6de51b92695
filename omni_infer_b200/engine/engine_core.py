"""Engine core: request intake -> scheduler -> worker -> outputs, with multi-step and asynchronous
scheduling (the reference patches these into its host engine: async_schedule_update_output.patch,
multi_step.patch, manual_apiserver_scaleout.patch)."""
from __future__ import annotations

import itertools
import logging
import os
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..adaptors.vllm.model_runner import RunnerConfig
from ..adaptors.vllm.worker import B200Worker
from ..models.config import ModelConfig, get_config
from .kv_manager import KVCacheManager
from .request import Request, RequestOutput, SamplingParams
from .scheduler import Scheduler, SchedulerConfig

logger = logging.getLogger("omni_infer_b200.engine")


@dataclass
class EngineConfig:
    model: str = "tiny-deepseek-v3"
    model_overrides: dict = field(default_factory=dict)
    device: Optional[str] = None
    tp_size: int = 1
    pp_size: int = 1                 # pipeline stages; every stage of a pipeline is given the same requests
    dense_mlp_tp_size: int = 1       # dense MLP layers + shared expert sharded over sub-groups of this size
    o_proj_tp_size: int = 1          # o_proj sharded over sub-groups of this size (attention data parallel)
    shared_expert_ranks: int = 0     # first N ranks hold only the shared expert, routed experts on the others
    vocab_parallel: bool = False     # embedding table + LM head sharded by vocabulary rows over all ranks
    scheduling_policy: str = "fcfs"  # fcfs | priority (smaller value first; decides admission order and who is preempted)
    block_size: int = 128
    num_kv_blocks: int = 0
    gpu_memory_utilization: float = 0.9
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 4096
    num_speculative_tokens: int = 0
    num_step: int = 1
    async_schedule: bool = False
    enable_prefix_caching: bool = False
    enable_chunked_prefill: bool = os.environ.get("FORCE_ENABLE_CHUNK_PREFILL", "0") == "1"
    decode_gear_list: list = field(default_factory=list)
    enforce_eager: bool = False
    ep_backend: str = "fused"
    attn_tp: bool = False            # tensor-parallel attention over all ranks (default: data-parallel attention)
    tp_backend: str = "fused"        # fused (GEMMs with the collectives inside) | nvls (same, reductions inside the NVSwitch) | nccl (library collectives)
    seed: int = 0
    kv_transfer_config: Optional[dict] = None    # {"kv_role": "kv_producer"|"kv_consumer", ...}
    enable_omni_attn: bool = False
    omni_attn_config: Optional[dict] = None
    placement_config: Optional[dict] = None
    eos_token_id: Optional[int] = None
    # per-rank state kept across restarts (KV block count, captured graph buckets, placement pattern and load history)
    state_dir: Optional[str] = os.environ.get("OMNI_STATE_DIR") or None


class EngineCore:
    def __init__(self, cfg: EngineConfig, model_cfg: Optional[ModelConfig] = None, weights=None, planner=None,
                 kv_connector_pair=None):
        self.cfg = cfg
        self.model_cfg = model_cfg or get_config(cfg.model, **cfg.model_overrides)
        if cfg.shared_expert_ranks:
            self.model_cfg.shared_expert_ranks = int(cfg.shared_expert_ranks)
        rc = RunnerConfig(block_size=cfg.block_size, num_kv_blocks=cfg.num_kv_blocks,
                          gpu_memory_utilization=cfg.gpu_memory_utilization, max_num_seqs=cfg.max_num_seqs,
                          max_model_len=cfg.max_model_len, max_num_batched_tokens=cfg.max_num_batched_tokens,
                          num_speculative_tokens=cfg.num_speculative_tokens, decode_gear_list=cfg.decode_gear_list,
                          enforce_eager=cfg.enforce_eager, seed=cfg.seed, ep_backend=cfg.ep_backend,
                          attn_tp=cfg.attn_tp, tp_backend=cfg.tp_backend, vocab_parallel=cfg.vocab_parallel)
        sched_conn = worker_conn = None
        if kv_connector_pair is not None:
            sched_conn, worker_conn = kv_connector_pair
        elif cfg.kv_transfer_config:
            from ..accelerators.pd import create_connectors
            sched_conn, worker_conn = create_connectors(cfg.kv_transfer_config, block_size=cfg.block_size)
        self.worker = B200Worker(self.model_cfg, rc, tp_size=cfg.tp_size, device=cfg.device, planner=planner,
                                 kv_connector=worker_conn, dense_mlp_tp_size=cfg.dense_mlp_tp_size,
                                 o_proj_tp_size=cfg.o_proj_tp_size, pp_size=cfg.pp_size)
        self.worker.init_device()
        self.state = None
        if cfg.state_dir:
            from ..parallel import get_parallel_state as _ps
            from .state_dir import StateDir, fingerprint
            self.state = StateDir(cfg.state_dir, _ps().rank, fingerprint(self.model_cfg, cfg, _ps().world_size))
        if planner is None and cfg.placement_config:
            # the planner sizes its slot tables from the world size, so it is built after the process group exists
            from ..accelerators.placement import OmniPlanner
            pc = dict(cfg.placement_config)
            saved = self.state.get_array("placement_pattern") if self.state is not None else None
            if saved is not None and not pc.get("pattern_path"):
                pc["pattern"] = saved          # the placement the previous run had arrived at
            planner = OmniPlanner.from_config(pc, self.model_cfg)
            self.worker.planner = self.worker.runner.planner = planner
        self.planner = planner
        self.worker.load_model(weights, seed=cfg.seed)
        if self.state is not None and not rc.num_kv_blocks and self.state.get("num_kv_blocks"):
            rc.num_kv_blocks = int(self.state.get("num_kv_blocks"))      # skips the profile run; ranks still agree on the minimum
        n_blocks = self.worker.determine_available_memory()
        self.worker.initialize_cache(n_blocks)
        self.worker.compile_or_warm_up_model()
        if self.state is not None:
            graphs = getattr(self.worker.runner, "graphs", None)
            self.state.save(num_kv_blocks=int(n_blocks),
                            graph_buckets=sorted(getattr(graphs, "graphs", {}).keys()) if graphs is not None else [])
            ema = self.state.get_array("placement_ema")
            if planner is not None and ema is not None:
                # handed to the balancer when the dynamic machinery is built
                planner.pending_ema = (self.state.get_array("placement_positions"), ema)
        self.kv = KVCacheManager(n_blocks, cfg.block_size, cfg.enable_prefix_caching)
        if cfg.enable_omni_attn:
            from ..accelerators.cache import apply_omni_attn_patch
            apply_omni_attn_patch(self, cfg.omni_attn_config or {})
        sc = SchedulerConfig(max_num_seqs=cfg.max_num_seqs, max_num_batched_tokens=cfg.max_num_batched_tokens,
                             max_model_len=cfg.max_model_len, num_speculative_tokens=cfg.num_speculative_tokens,
                             num_step=cfg.num_step, async_schedule=cfg.async_schedule,
                             enable_chunked_prefill=cfg.enable_chunked_prefill, policy=cfg.scheduling_policy)
        self.scheduler = Scheduler(sc, self.kv, connector=sched_conn)
        self._ids = itertools.count()
        from ..parallel import get_parallel_state
        self._world = get_parallel_state().world_size
        self._pool = ThreadPoolExecutor(max_workers=1) if cfg.async_schedule else None
        self._inflight = None
        self._deferred_aborts: list = []
        self.metrics = {"steps": 0, "prefill_steps": 0, "decode_steps": 0, "generated_tokens": 0}

    # ------------------------------------------------------------------ intake
    def save_state(self) -> None:
        """Writes what a restart can reuse (called at shutdown, and by whoever wants a checkpoint in between)."""
        if self.state is None:
            return
        if self.planner is not None:
            self.state.save(**self.planner.export_state())

    @property
    def role(self) -> str:
        kv_role = (self.cfg.kv_transfer_config or {}).get("kv_role", "")
        return {"kv_producer": "prefill", "kv_consumer": "decode"}.get(kv_role, "mixed")

    def add_request(self, prompt_token_ids, sampling: Optional[SamplingParams] = None, request_id: Optional[str] = None,
                    kv_transfer_params: Optional[dict] = None, priority: int = 0) -> str:
        rid = request_id or f"req-{next(self._ids)}"
        vocab = self.model_cfg.vocab_size
        prompt_token_ids = list(prompt_token_ids)
        if prompt_token_ids and not (min(prompt_token_ids) >= 0 and max(prompt_token_ids) < vocab):
            # the embedding lookup trusts its indices: an id outside the table must never reach the device
            raise ValueError(f"prompt token ids must lie in [0, {vocab})")
        req = Request(rid, prompt_token_ids, sampling or SamplingParams(), priority=priority,
                      eos_token_id=self.cfg.eos_token_id, kv_transfer_params=kv_transfer_params, role=self.role)
        if not self.scheduler.try_pull_kv_fast_path(req):
            self.scheduler.add_request(req)
        else:
            self.scheduler.requests[rid] = req
            self.scheduler.waiting.append(req)
        return rid

    def abort(self, request_id: str) -> None:
        """Drops a request.  While a round is being executed on the worker thread (asynchronous scheduling) the runner
        reads the requests of that round - their block lists, their token counts - so the drop waits until the round's
        results have been applied; the request takes part in at most that one more round."""
        if self._inflight is not None:
            self._deferred_aborts.append(request_id)
            return
        self.scheduler.abort_request(request_id)

    @property
    def has_unfinished(self) -> bool:
        # an empty round in flight (an idle rank keeping step with its peers) is not work of this rank
        return self.scheduler.has_unfinished or (self._inflight is not None and not self._inflight[0].empty)

    # ------------------------------------------------------------------ stepping
    def step(self) -> list:
        if self.cfg.async_schedule:
            return self.step_async()
        so = self.scheduler.schedule()
        # data-parallel ranks step together: an idle rank runs a padded dummy batch so that the
        # expert-parallel exchanges of the busy ranks find their peer
        out = self._execute(so)
        res = self.scheduler.update_from_output(so, out)
        self._account(so, res)
        return res

    def step_async(self) -> list:
        """Overlap: while the worker executes round N, apply round N-1's results and schedule round N+1.
        A request scheduled twice in flight would need tokens the host has not seen yet, so a request
        takes part in at most one in-flight round; with enough running requests the device never idles."""
        results: list = []
        if self._inflight is None:
            so = self.scheduler.schedule()
            self._inflight = (so, self._pool.submit(self._execute, so))
            return results
        so, fut = self._inflight
        out = fut.result()
        res = self.scheduler.update_from_output(so, out)
        self._account(so, res)
        self._inflight = None
        for rid in self._deferred_aborts:          # nothing is executing now: requests may change
            self.scheduler.abort_request(rid)
        self._deferred_aborts = []
        nxt = self.scheduler.schedule()
        # with several data-parallel ranks an idle rank keeps executing (dummy batches): its peers' exchanges need it
        if not nxt.empty or self._world > 1 or nxt.kv_connector_metadata is not None and self.scheduler.has_unfinished:
            self._inflight = (nxt, self._pool.submit(self._execute, nxt))
        else:
            self._inflight = None
        return res

    def _execute(self, so):
        """One round on the worker; a rank with nothing scheduled still takes part in the step of its peers."""
        if so.empty and self._world > 1:
            self.worker.execute_dummy_batch()
        return self.worker.execute_model(so)

    def _account(self, so, res) -> None:
        self.metrics["steps"] += 1
        self.metrics["prefill_steps" if so.is_prefill else "decode_steps"] += 0 if so.empty else 1
        self.metrics["generated_tokens"] += sum(len(r.new_token_ids) for r in res)

    @property
    def peers_busy(self) -> bool:
        """With several data-parallel ranks: did any rank report live requests in the last step's agreement?"""
        return self._world > 1 and bool(getattr(self.worker.runner, "peers_busy", False))

    def run_until_done(self, max_steps: int = 1_000_000) -> dict:
        """Step until this rank has nothing left; with several data-parallel ranks, until no rank has (an idle rank
        keeps stepping with dummy batches so that its peers' expert-parallel exchanges complete).  Every rank sees the
        same agreement, so all of them leave the loop after the same step."""
        outs: dict = {}
        for _ in range(max_steps):
            if not self.has_unfinished and self._world == 1:
                break
            for r in self.step():
                outs.setdefault(r.request_id, []).extend(r.new_token_ids)
            if self._world > 1 and not self.has_unfinished and not self.peers_busy:
                break
        return outs


class LLM:
    """Offline front end: ``LLM(...).generate(list_of_token_id_lists, SamplingParams)``."""

    def __init__(self, model: str = "tiny-deepseek-v3", **kw):
        model_cfg = kw.pop("model_config", None)
        weights = kw.pop("weights", None)
        self.engine = EngineCore(EngineConfig(model=model, **kw), model_cfg=model_cfg, weights=weights)

    def generate(self, prompts: list, sampling: Optional[SamplingParams] = None) -> list:
        ids = [self.engine.add_request(p, sampling) for p in prompts]
        outs = self.engine.run_until_done()
        return [outs.get(i, []) for i in ids]
