"""Model runner: turns a SchedulerOutput into device work.

Counterpart of the reference's NPUModelRunner (omni/adaptors/vllm/worker/npu_model_runner.py:120-995):
``_prepare_inputs`` (positions, slot mapping, attention state, padding the decode batch to a "gear"),
the multi-step loop with on-device input advance, logits -> sampler or MTP verification -> ``run_mtp``
drafting, KV-connector hooks, the OmniPlacement hook between steps, ``load_model`` (main model + up to
three MTP drafters sharing embedding and LM head), ``initialize_kv_cache``, ``capture_model`` and
``_get_closest_gear``.  The vendor graph compiler's gears become CUDA-graph buckets
(:mod:`omni_infer_b200.adaptors.vllm.cuda_graphs`).
"""
from __future__ import annotations

import logging
import os
import time
from dataclasses import dataclass, field
from typing import Optional

import torch

from ... import ops
from ...engine.request import ModelRunnerOutput, SchedulerOutput
from ...layers.common import AttnMetadata
from ...models import build_model
from ...models.config import ModelConfig
from ...parallel import get_parallel_state

logger = logging.getLogger("omni_infer_b200.runner")


@dataclass
class RunnerConfig:
    block_size: int = 128
    num_kv_blocks: int = 0                     # 0 = size from free memory
    gpu_memory_utilization: float = 0.9
    max_num_seqs: int = 256
    max_model_len: int = 4096
    max_num_batched_tokens: int = 8192
    num_speculative_tokens: int = 0
    decode_gear_list: list = field(default_factory=list)   # CUDA-graph batch buckets; [] = powers of two
    use_cuda_graph: bool = True
    enforce_eager: bool = False
    seed: int = 0
    kv_cache_dtype: str = "auto"
    control_accept_rate: float = -1.0          # test knob of the MTP verifier (reference: model_extra_config)
    ep_backend: str = "fused"                  # fused (NVLink peer-memory kernels) | nccl (all-to-all baseline)
    ep_wait_ms: float = 2000.0                 # bound of every cross-rank wait inside the fused kernels
    attn_tp: bool = False                      # attention heads sharded over all ranks, token-sharded hidden states
    tp_backend: str = "fused"                  # fused | nvls | nccl
    vocab_parallel: bool = False               # embedding table and LM head sharded by vocabulary rows over all ranks
    # how long a rank waits for its peers in the per-step host agreement once serving has begun (start-up, where ranks
    # may be minutes apart, uses the process group's own limit): a peer that has died or stopped stepping then ends
    # this rank's step with an error instead of holding it for the group's ten minutes
    agree_timeout_s: float = float(os.environ.get("OMNI_AGREE_TIMEOUT_S", "120"))


class ModelRunner:
    def __init__(self, model_cfg: ModelConfig, cfg: RunnerConfig, device: torch.device, planner=None,
                 kv_connector=None):
        self.model_cfg, self.cfg, self.device = model_cfg, cfg, device
        self.planner = planner
        self.kv_connector = kv_connector
        self.model = None
        self.drafters: list = []
        self.kv_caches: list = []
        self.drafter_kv: list = []
        self.graphs = None
        self.rng = torch.Generator(device=device)
        self.rng.manual_seed(cfg.seed)
        self.tpr = 1 + cfg.num_speculative_tokens
        self._bt_width = (cfg.max_model_len + cfg.block_size - 1) // cfg.block_size + 1
        self.step_times: list = []
        self.omni = None
        self._agreements_done = 0      # per-step host agreements completed (the first ones belong to start-up)

    # ------------------------------------------------------------------ model / cache set-up
    def load_model(self, weights=None, seed: Optional[int] = 0) -> None:
        cfg = self.model_cfg
        t0 = time.time()
        self.setup_tensor_parallel()
        self.model = build_model(cfg, device=self.device, planner=self.planner,
                                 seed=seed if weights is None else None)
        from ...models.deepseek_mtp import DeepseekV3MTP
        n_draft = min(self.cfg.num_speculative_tokens, max(cfg.num_nextn_predict_layers, 0), 3)
        if self.cfg.num_speculative_tokens and get_parallel_state().pp_size > 1:
            raise ValueError("MTP drafting is not combined with pipeline parallelism")
        if self.cfg.num_speculative_tokens and n_draft == 0:
            raise ValueError("speculative decoding needs num_nextn_predict_layers > 0 in the model config")
        for i in range(n_draft):
            d = DeepseekV3MTP(cfg, self.model, mtp_index=i, device=self.device)
            if weights is None:
                from ...quantization.loader import init_random_weights
                init_random_weights(d, (seed or 0) + 1000 + i)
            self.drafters.append(d)
        if weights is not None:
            wl = list(weights) if self.drafters else weights
            self.model.load_weights(wl, planner=self.planner)
            for d in self.drafters:
                d.load_weights(wl, planner=self.planner)
        if self.planner is not None:
            self.planner.init_dram_weights(self.model)
        self.setup_expert_parallel()
        logger.info("model %s loaded in %.1fs", cfg.name or cfg.architecture, time.time() - t0)

    def setup_tensor_parallel(self) -> None:
        """Tensor-parallel attention: every rank runs the same batch, heads are sharded, and the row all-gather /
        reduce-scatter around the attention block run inside the GEMMs (parallel/tp_fused.py)."""
        ps = get_parallel_state()
        cfg = self.model_cfg
        if self.cfg.vocab_parallel and ps.world_size > 1:
            # every rank must enter the table / head collectives in every step: true for expert-parallel models (idle
            # ranks run dummy batches) and for tensor-parallel attention, not for independent dense replicas
            if ps.pp_size > 1 or not (cfg.is_moe or self.cfg.attn_tp):
                raise ValueError("vocab_parallel needs ranks that step together (an expert-parallel model or attn_tp) and no "
                                 "pipeline stages")
            cfg.vocab_parallel_size, cfg.vocab_parallel_rank = ps.world_size, ps.rank
        if not self.cfg.attn_tp or ps.world_size == 1:
            return
        assert cfg.architecture.startswith(("Deepseek", "Qwen")), "tensor-parallel attention is wired for the MLA and GQA models"
        if not cfg.use_mla:
            from ...layers.gqa import shard_heads
            shard_heads(cfg.num_attention_heads, cfg.num_key_value_heads, ps.world_size, ps.rank)   # raises if it cannot
        cfg.attn_tp_size, cfg.attn_tp_rank = ps.world_size, ps.rank
        from ...parallel.tp_fused import TpFusedContext, TpNcclBaseline
        grp = ps.group("world").group
        if self.cfg.tp_backend in ("fused", "nvls") and self.device.type == "cuda":
            max_tok = max(self.cfg.max_num_batched_tokens, self.cfg.max_num_seqs * self.tpr) + 4 * ps.world_size
            # "nvls": the reducing collectives go through the NVSwitch's in-switch reduction (multimem)
            ps.tp_fused = TpFusedContext(grp, max_tokens=max_tok, max_k_bytes=cfg.hidden_size * 2, max_n=cfg.hidden_size,
                                         wait_ms=self.cfg.ep_wait_ms, nvls=self.cfg.tp_backend == "nvls")
        else:
            ps.tp_fused = TpNcclBaseline(grp)

    def setup_expert_parallel(self) -> None:
        """With more than one rank the routed experts are sharded over all ranks.  Decode-sized batches go
        through the fused NVLink dispatch/combine kernels (e4m3 rows for e4m3 experts, bf16 rows otherwise),
        anything larger through the all-to-all baseline.  All ranks must take the same path in a step, so the choice is
        agreed on the host group before every forward (:meth:`_agree_ep_path`)."""
        self.ep_ctx = None
        ps = get_parallel_state()
        cfg = self.model_cfg
        if ps.world_size == 1 or not cfg.is_moe:
            return
        moe_layers = [m for m in self.model.modules() if m.__class__.__name__ == "MoELayer"]
        for d in self.drafters:
            moe_layers += [m for m in d.modules() if m.__class__.__name__ == "MoELayer"]
        self._moe_layers = moe_layers
        if (self.cfg.ep_backend == "fused" and self.device.type == "cuda" and cfg.dtype == "bfloat16"
                and cfg.hidden_size % 128 == 0 and ps.pp_size == 1):
            from ...parallel.ep_fused import EpContext
            # e4m3 experts: rows are dispatched quantised (1x128 scales); unquantised experts: bf16 rows as they are
            # with dedicated shared-expert ranks every token also sends one row per shared piece
            top_k = cfg.num_experts_per_tok + (moe_layers[0].shared_pieces if moe_layers else 0)
            self.ep_ctx = EpContext(cfg.hidden_size, top_k, self.cfg.max_num_seqs * self.tpr,
                                    wait_ms=self.cfg.ep_wait_ms, payload="fp8" if cfg.quantization == "fp8_block" else "bf16")
            self.ep_max_tokens = self.ep_ctx.max_tokens

    def _agree_start(self, num_tokens: int, rounds: int, has_work: bool):
        """Start the per-step agreement of the data-parallel ranks (host group, asynchronous so that it overlaps
        the input preparation).  Every rank contributes its token rows, the model rounds its batch needs (a prefill
        is one round, a decode ``num_step``) and whether it has live requests.  The reference keeps its DP ranks in
        step the same way, with a MAX all-reduce of the token count on the CPU group
        (omni/adaptors/vllm/worker/npu_model_runner.py:989-995)."""
        ps = get_parallel_state()
        # every rank must take the same decision here, whatever layers it happens to hold (pipeline stages)
        if ps.world_size == 1 or not self.model_cfg.is_moe:
            return None
        import torch.distributed as dist
        # fourth value: minus the number of placement rounds this rank has complete, so that the MAX gives the minimum
        # over the ranks - a round is applied in the step in which every rank has it (see _place_experts)
        ready = self.planner.ready_rounds() if self.planner is not None else 0
        t = torch.tensor([num_tokens, rounds, 1 if has_work else 0, -ready], dtype=torch.int64)
        work = dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ps.group("cpu").group, async_op=True)
        return t, work

    def _agree_finish(self, handle, rounds: int = 1) -> int:
        """Finish the agreement: choose the expert-parallel path every rank takes in this step (the fused peer-memory
        kernels only if every rank's rows fit their buffers and nothing forces the baseline) and return the number of
        model rounds all ranks run.  ``peers_busy`` tells the engine loop whether any rank still has requests."""
        ps = get_parallel_state()
        if handle is None:
            self._place_experts(None)
            self.peers_busy = False
            self._ep_fused_now = getattr(self, "ep_ctx", None) is not None
            ps.step_max_tokens = 0
            return rounds
        t, work = handle
        if self._agreements_done and self.cfg.agree_timeout_s > 0:
            import datetime
            try:
                ok = work.wait(timeout=datetime.timedelta(seconds=self.cfg.agree_timeout_s))
            except RuntimeError as e:
                raise RuntimeError(f"a peer rank did not join the step agreement within {self.cfg.agree_timeout_s:.0f} s "
                                   f"(it has died or stopped stepping): {e}") from e
            if ok is False:
                raise RuntimeError(f"a peer rank did not join the step agreement within {self.cfg.agree_timeout_s:.0f} s")
        else:
            work.wait()
        self._agreements_done += 1
        max_tokens, max_rounds, any_work = int(t[0]), int(t[1]), bool(int(t[2]))
        self._place_experts(-int(t[3]))
        self.peers_busy = any_work
        ps.step_max_tokens = max_tokens        # layers sharded over a sub-group pad their rows to this
        ctx = getattr(self, "ep_ctx", None)
        fused = ctx is not None and max_tokens <= self.ep_max_tokens and not getattr(self, "force_ep_baseline", False)
        self._ep_fused_now = fused
        for m in getattr(self, "_moe_layers", ()):
            m.ep_ctx = ctx if fused else None
        return max(rounds, max_rounds)

    def _place_experts(self, min_ready) -> None:
        """Between two steps, right after the ranks' agreement: apply the expert moves of a finished placement round.
        ``min_ready`` is the smallest number of complete rounds on any rank, so every rank applies a round in the same
        step; a rank that switched its selector to a replica before the holder has copied the weights in would send
        tokens to an empty slot.  (One rank alone passes None and goes by its own counter.)"""
        if self.planner is not None:
            self.planner.place_experts(min_ready)

    def _agree_ep_path(self, num_tokens: int, rounds: int = 1, has_work: bool = True) -> int:
        return self._agree_finish(self._agree_start(num_tokens, rounds, has_work), rounds)

    def _dummy_rounds(self, n: int) -> None:
        """Extra rounds with no live row, so that this rank makes as many expert-parallel exchanges as the rank with
        the most rounds: one main-model forward and one forward per drafter each."""
        if n <= 0:
            return
        padded = self._get_closest_gear(1) if self.graphs is not None else 1
        ids, md = self._prepare_decode(SchedulerOutput([], False), padded)
        md.num_valid = self._to_dev([0], torch.int32)
        for _ in range(n):
            hidden, _ = self._forward_decode(ids, md, padded)
            h = hidden
            for di, d in enumerate(self.drafters):
                h = d(ids, md, self.drafter_kv[di], h)
                if self.model_cfg.vocab_parallel_size > 1:
                    d.compute_logits(h[:1])      # the sharded head is a collective: join the live ranks' call

    def kv_bytes_per_block(self) -> int:
        cfg = self.model_cfg
        layers = self.model.num_kv_layers + len(self.drafters)
        esz = 4 if cfg.dtype == "float32" else 2
        return layers * self.cfg.block_size * cfg.kv_bytes_per_token(esz)

    def determine_num_blocks(self) -> int:
        if self.cfg.num_kv_blocks:
            return self.cfg.num_kv_blocks
        if self.device.type != "cuda":
            return 256
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - int(total * (1.0 - self.cfg.gpu_memory_utilization))
        return max(16, int(budget // self.kv_bytes_per_block()))

    def initialize_kv_cache(self, num_blocks: int) -> None:
        cfg, bs = self.model_cfg, self.cfg.block_size
        dt = self.model.model.dtype if hasattr(self.model, "model") else torch.bfloat16
        self.num_blocks = num_blocks

        ipc = (self.kv_connector is not None and getattr(self.kv_connector, "transport", "inproc") != "inproc"
               and self.device.type == "cuda")

        def zeros(*shape):
            if ipc:     # another process will open this memory through CUDA IPC
                from ...parallel.symmetric_heap import alloc_ipc_tensor
                return alloc_ipc_tensor(shape, dt)
            return torch.zeros(*shape, dtype=dt, device=self.device)

        def one():
            if cfg.use_mla:
                return zeros(num_blocks, bs, cfg.kv_lora_rank + cfg.qk_rope_head_dim)
            return (zeros(num_blocks, bs, cfg.local_kv_heads, cfg.head_dim),
                    zeros(num_blocks, bs, cfg.local_kv_heads, cfg.head_dim))

        self.kv_caches = [one() for _ in range(self.model.num_kv_layers)]
        self.drafter_kv = [[one()] for _ in self.drafters]
        if self.kv_connector is not None:
            self.kv_connector.register_kv_caches(self.kv_caches + [k[0] for k in self.drafter_kv])

    def enable_omni_attn(self, state, num_window_blocks: int) -> None:
        """Compressed layers get a cache of per-request windows; decode runs eagerly from here on."""
        cfg, bs = self.model_cfg, self.cfg.block_size
        self.omni = state
        dt = self.model.model.dtype
        ipc = (self.kv_connector is not None and getattr(self.kv_connector, "transport", "inproc") != "inproc"
               and self.device.type == "cuda")

        def zeros(*shape):
            if ipc:     # a prefill instance in another process writes the transferred windows through CUDA IPC
                from ...parallel.symmetric_heap import alloc_ipc_tensor
                return alloc_ipc_tensor(shape, dt)
            return torch.zeros(*shape, dtype=dt, device=self.device)

        compressed = []
        for i in range(self.model.num_kv_layers):
            if not state.is_compressed(i):
                continue
            compressed.append(i)
            if cfg.use_mla:
                self.kv_caches[i] = zeros(num_window_blocks, bs, cfg.kv_lora_rank + cfg.qk_rope_head_dim)
            else:
                self.kv_caches[i] = tuple(zeros(num_window_blocks, bs, cfg.local_kv_heads, cfg.head_dim) for _ in range(2))
        self.graphs = None
        if self.kv_connector is not None:
            # the connector keeps the cache tensors: tell it about the new ones and which layers they belong to
            self.kv_connector.register_kv_caches(self.kv_caches + [k[0] for k in self.drafter_kv], compressed_layers=compressed)
            self.kv_connector.omni_spec = state.spec

    # ------------------------------------------------------------------ gears / graphs
    def gear_list(self) -> list:
        if self.cfg.decode_gear_list:
            return sorted(set(int(g) for g in self.cfg.decode_gear_list))
        gears, g = [], 1
        while g < self.cfg.max_num_seqs:
            gears.append(g)
            g *= 2
        gears.append(self.cfg.max_num_seqs)
        return gears

    def _get_closest_gear(self, n: int) -> int:
        for g in self.gear_list():
            if g >= n:
                return g
        return n

    def capture_model(self) -> None:
        """Capture one CUDA graph per decode bucket, largest first so smaller ones reuse its memory pool."""
        if self.device.type != "cuda" or not self.cfg.use_cuda_graph or self.cfg.enforce_eager:
            return
        if get_parallel_state().pp_size > 1:
            logger.info("pipeline parallelism: stages hand over hidden states with point-to-point sends; decode stays eager")
            return
        if get_parallel_state().world_size > 1 and self.model_cfg.is_moe and getattr(self, "ep_ctx", None) is None:
            logger.info("expert parallelism over NCCL all-to-all needs host-side split sizes: decode stays eager")
            return
        tpc = get_parallel_state().tp_fused
        if tpc is not None and tpc.__class__.__name__ == "TpNcclBaseline":
            logger.info("tensor-parallel attention over library collectives: decode stays eager")
            return
        from .cuda_graphs import DecodeGraphs
        self.graphs = DecodeGraphs(self)
        t0 = time.time()
        for g in reversed(self.gear_list()):
            self.graphs.capture(g)
        logger.info("captured %d decode graphs in %.1fs", len(self.gear_list()), time.time() - t0)

    # ------------------------------------------------------------------ input preparation
    def _slots(self, block_ids: list, start: int, n: int) -> list:
        bs = self.cfg.block_size
        return [block_ids[p // bs] * bs + p % bs for p in range(start, start + n)]

    def _to_dev(self, data, dtype) -> torch.Tensor:
        t = torch.tensor(data, dtype=dtype)
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def _prepare_prefill(self, so: SchedulerOutput):
        ids, pos, slots, cu_q, cu_k, qlens, ctx, sample_idx, seq_lens = [], [], [], [0], [0], [], [], [], []
        gather, need_gather = [], False
        bt_rows = []
        for s in so.scheduled:
            r = s.request
            st, n = r.num_computed_tokens, s.num_scheduled_tokens
            toks = r.all_token_ids[st:st + n]
            ids += toks
            pos += list(range(st, st + n))
            slots += self._slots(r.block_ids, st, n)
            cu_q.append(cu_q[-1] + n)
            cu_k.append(cu_k[-1] + st + n)
            qlens.append(n)
            ctx.append(st)
            seq_lens.append(st + n)
            need_gather |= st > 0
            gather += self._slots(r.block_ids, 0, st + n)
            sample_idx.append(cu_q[-1] - 1)
            bt_rows.append(r.block_ids + [0] * (self._bt_width - len(r.block_ids)))
        md = AttnMetadata(
            is_prefill=True, positions=self._to_dev(pos, torch.int64), slot_mapping=self._to_dev(slots, torch.int64),
            block_table=self._to_dev(bt_rows, torch.int32), seq_lens=self._to_dev(seq_lens, torch.int32),
            cu_q=self._to_dev(cu_q, torch.int32), cu_k=self._to_dev(cu_k, torch.int32), query_lens=qlens,
            context_lens=ctx, max_q=max(qlens), max_k=max(seq_lens),
            kv_gather_slots=self._to_dev(gather, torch.int64) if need_gather else None,
            sample_indices=self._to_dev(sample_idx, torch.int64))
        if self.omni is not None:
            oslots = []
            for s in so.scheduled:
                r = s.request
                oslots += self.omni.prefill_slots(r.omni_block_ids, r.num_computed_tokens, s.num_scheduled_tokens,
                                                  r.num_prompt_tokens, total_len=r.num_tokens)
            md.omni = {"pattern": self.omni.pattern, "slot_mapping": self._to_dev(oslots, torch.int64)}
        return self._to_dev(ids, torch.int64), md

    def _prepare_decode(self, so: SchedulerOutput, padded: int):
        """Decode inputs for ``padded`` rows (live requests first).  Everything is assembled with numpy in
        one pinned staging buffer and moved with a single host->device copy."""
        import numpy as np

        tpr, bs, W = self.tpr, self.cfg.block_size, self._bt_width
        B = len(so.scheduled)
        n = padded * tpr
        # int64 section: ids | positions | slots ; int32 section: q_seq_lens | seq_lens | q_to_seq | num_valid | block table
        n64 = 3 * n
        n32 = n + padded + n + 2 + padded * W
        total_bytes = n64 * 8 + n32 * 4
        key = (padded, tpr)
        stage = getattr(self, "_stage", None)
        if stage is None or stage[0] != key:
            host = torch.empty(total_bytes, dtype=torch.uint8)
            if self.device.type == "cuda":
                host = host.pin_memory()
            self._stage = stage = (key, host, host.numpy())
        _, host, raw = stage
        a64 = raw[: n64 * 8].view(np.int64)
        a32 = raw[n64 * 8:].view(np.int32)
        ids, pos, slots = a64[:n].reshape(padded, tpr), a64[n:2 * n].reshape(padded, tpr), a64[2 * n:].reshape(padded, tpr)
        o = 0
        qlens = a32[o:o + n].reshape(padded, tpr); o += n
        seq_lens = a32[o:o + padded]; o += padded
        q_to_seq = a32[o:o + n]; o += n
        num_valid = a32[o:o + 2]; o += 2
        bt = a32[o:o + padded * W].reshape(padded, W)
        ids[:] = 0
        bt[:] = 0
        st = np.zeros(padded, dtype=np.int64)
        for i, s in enumerate(so.scheduled):
            r = s.request
            c = r.num_computed_tokens
            st[i] = c
            npt = len(r.prompt_token_ids)
            ids[i, 0] = r.output_token_ids[c - npt] if c >= npt else r.prompt_token_ids[c]
            if s.spec_token_ids:
                k = min(len(s.spec_token_ids), tpr - 1)
                ids[i, 1:1 + k] = s.spec_token_ids[:k]
            nb = len(r.block_ids)
            bt[i, :nb] = r.block_ids
        j = np.arange(tpr, dtype=np.int64)[None, :]
        pos[:] = st[:, None] + j
        live = np.arange(padded) < B
        blk = np.take_along_axis(bt.astype(np.int64), np.minimum(pos // bs, W - 1), axis=1)
        slots[:] = np.where(live[:, None], blk * bs + pos % bs, -1)
        pos[~live] = 0
        qlens[:] = np.where(live[:, None], pos + 1, 0)
        seq_lens[:] = np.where(live, st + tpr, 0)
        q_to_seq[:] = np.repeat(np.arange(padded, dtype=np.int32), tpr)
        num_valid[0] = B * tpr
        max_seq = int(seq_lens.max()) if B else 0
        dev = host.to(self.device, non_blocking=True) if self.device.type == "cuda" else host.clone()
        d64 = dev[: n64 * 8].view(torch.int64)
        d32 = dev[n64 * 8:].view(torch.int32)
        o = 0
        d_q = d32[o:o + n]; o += n
        d_seq = d32[o:o + padded]; o += padded
        d_q2s = d32[o:o + n]; o += n
        d_nv = d32[o:o + 1]; o += 2
        d_bt = d32[o:o + padded * W].view(padded, W)
        md = AttnMetadata(
            is_prefill=False, positions=d64[n:2 * n], slot_mapping=d64[2 * n:3 * n], block_table=d_bt, seq_lens=d_seq,
            tokens_per_req=tpr, q_seq_lens=d_q, q_to_seq=d_q2s, max_seq_len=max_seq,
            num_valid=d_nv if padded != B else None)
        if self.omni is not None:
            nb = self.omni.spec.blocks_per_request
            wt = [list(s.request.omni_block_ids) for s in so.scheduled] + [[0] * nb] * (padded - B)
            pl = [s.request.num_prompt_tokens for s in so.scheduled] + [0] * (padded - B)
            pl_dev = self._to_dev(pl, torch.int32)
            om = self.omni.decode_metadata(d_seq, pl_dev, self._to_dev(wt, torch.int32))
            om["pattern"], om["prompt_lens"] = self.omni.pattern, pl_dev
            md.omni = om
        return d64[:n], md

    # ------------------------------------------------------------------ sampling
    def _penalise(self, logits: torch.Tensor, reqs: list, rows_per_req: int) -> torch.Tensor:
        """Repetition / frequency / presence penalties of the requests that ask for them; every row of a request
        (its verified token and its draft positions) sees the request's token history."""
        if not any(r.sampling.has_penalties for r in reqs):
            return logits
        n = logits.shape[0]
        width = max(r.num_tokens for r in reqs)
        hist = torch.full((n, width), -1, dtype=torch.int32)
        npr = torch.zeros(n, dtype=torch.int32)
        rep, freq, pres = torch.ones(n), torch.zeros(n), torch.zeros(n)
        for i, r in enumerate(reqs):
            if not r.sampling.has_penalties:
                continue
            sl = slice(i * rows_per_req, (i + 1) * rows_per_req)
            toks = torch.tensor(r.all_token_ids, dtype=torch.int32)
            hist[sl, : toks.numel()] = toks
            npr[sl] = r.num_prompt_tokens
            rep[sl], freq[sl], pres[sl] = r.sampling.repetition_penalty, r.sampling.frequency_penalty, r.sampling.presence_penalty
        dev = self.device
        return ops.apply_penalties(logits, hist.to(dev), npr.to(dev), rep.to(dev), freq.to(dev), pres.to(dev))

    def _sample(self, logits: torch.Tensor, reqs: list, rows_per_req: int) -> torch.Tensor:
        """logits [len(reqs) * rows_per_req (+ padding), V] -> token ids (padding rows included)."""
        logits = self._penalise(logits, reqs, rows_per_req)
        if all(r.sampling.greedy for r in reqs):
            return ops.argmax(logits)
        n = logits.shape[0]
        temp = torch.zeros(n)
        tk = torch.zeros(n, dtype=torch.int32)
        tp = torch.ones(n)
        for i, r in enumerate(reqs):
            sl = slice(i * rows_per_req, (i + 1) * rows_per_req)
            temp[sl], tk[sl], tp[sl] = r.sampling.temperature, r.sampling.top_k, r.sampling.top_p
        u = torch.rand(n, device=self.device, generator=self.rng)
        return ops.sample_topk_topp(logits, temp.to(self.device), tk.to(self.device), tp.to(self.device), u)

    # ------------------------------------------------------------------ execution
    @torch.inference_mode()
    def execute_model(self, so: SchedulerOutput) -> ModelRunnerOutput:
        t0 = time.perf_counter()
        fin_send, fin_recv = set(), set()
        if self.kv_connector is not None:
            self.kv_connector.bind_connector_metadata(so.kv_connector_metadata)
            self.kv_connector.start_load_kv()
        if so.empty:
            failed = set()
            if self.kv_connector is not None:
                fin_send, fin_recv = self.kv_connector.get_finished(so.finished_req_ids)
                failed = self.kv_connector.take_failed()
            return ModelRunnerOutput([], [[]], None, fin_send, fin_recv, failed)
        reqs = [s.request for s in so.scheduled]
        if so.is_prefill:
            out = self._run_prefill(so, reqs)
        else:
            out = self._run_decode(so, reqs)
        if self.kv_connector is not None:
            self.kv_connector.wait_for_save()
            fin_send, fin_recv = self.kv_connector.get_finished(so.finished_req_ids)
            out.finished_sending, out.finished_recving = fin_send, fin_recv
            out.failed_recving = self.kv_connector.take_failed()
        out.step_time_s = time.perf_counter() - t0
        self.step_times.append(out.step_time_s)
        return out

    def _run_prefill(self, so, reqs) -> ModelRunnerOutput:
        handle = self._agree_start(sum(x.num_scheduled_tokens for x in so.scheduled), 1, True)
        ids, md = self._prepare_prefill(so)
        rounds = self._agree_finish(handle, 1)
        hidden = self.model(ids, md, self.kv_caches)
        pp = self._pipeline()
        if pp is None or pp.is_last:
            last_h = hidden[md.sample_indices]
            logits = self.model.compute_logits(last_h)
            toks = self._sample(logits, reqs, 1)
        else:
            toks = None
        if pp is not None:
            toks = pp.broadcast_tokens(toks, len(reqs), self.device)
        spec = None
        if self.drafters:
            # drafter prefill: tokens shifted left, the sampled token closes each request's row
            mtp_in = torch.empty_like(ids)
            mtp_in[:-1] = ids[1:]
            mtp_in[md.sample_indices] = toks
            spec_cols, h, cur = [], hidden, mtp_in
            for di, d in enumerate(self.drafters):
                h = d(cur, md, self.drafter_kv[di], h)
                dl = d.compute_logits(h[md.sample_indices])
                draft = ops.argmax(dl)
                spec_cols.append(draft)
                if di + 1 < len(self.drafters):
                    nxt = torch.empty_like(cur)
                    nxt[:-1] = cur[1:]
                    nxt[md.sample_indices] = draft
                    cur = nxt
            spec_t = torch.stack(spec_cols, dim=1).tolist()
            pad = self.cfg.num_speculative_tokens - len(self.drafters)
            spec = [row + [0] * pad for row in spec_t]
        self._dummy_rounds(rounds - 1)
        tl = toks.tolist()
        return ModelRunnerOutput([r.request_id for r in reqs], [[[t] for t in tl]], spec)

    def _forward_decode(self, ids, md, padded):
        """hidden, logits and greedy tokens for one decode step (CUDA graph replay when available)."""
        # a captured graph contains the fused exchange; when the ranks agreed on the baseline for this step (a peer
        # prefills more rows than the fused buffers hold) the step runs eagerly on the agreed path instead
        graph_ok = getattr(self, "_ep_fused_now", True) or getattr(self, "ep_ctx", None) is None
        cfg = self.model_cfg
        if getattr(cfg, "dense_mlp_tp_size", 1) > 1 or getattr(cfg, "o_proj_tp_size", 1) > 1:
            # sub-group collectives inside a graph have the captured row count: replay only when every rank runs it
            m = get_parallel_state().step_max_tokens
            graph_ok = graph_ok and (m == 0 or m == padded * self.tpr)
        if self.graphs is not None and self.graphs.has(padded) and graph_ok:
            return self.graphs.replay(padded, ids, md)
        hidden = self.model(ids, md, self.kv_caches)
        pp = self._pipeline()
        logits = self.model.compute_logits(hidden) if (pp is None or pp.is_last) else None
        return hidden, logits

    def _pipeline(self):
        """This rank's pipeline stage, or None without pipeline parallelism."""
        inner = getattr(self.model, "model", None)
        return getattr(inner, "pp", None)

    def _run_decode(self, so, reqs) -> ModelRunnerOutput:
        tpr, B = self.tpr, len(reqs)
        padded = self._get_closest_gear(B) if (self.graphs is not None) else B
        handle = self._agree_start(padded * tpr, so.num_step, True)
        ids, md = self._prepare_decode(so, padded)
        rounds = self._agree_finish(handle, so.num_step)
        steps_out: list = []
        spec_final = None
        for step in range(so.num_step):
            hidden, logits = self._forward_decode(ids, md, padded)
            pp = self._pipeline()
            toks = self._sample(logits, reqs, tpr) if logits is not None else None
            if pp is not None:
                toks = pp.broadcast_tokens(toks, padded * tpr, self.device)
            if tpr == 1:
                steps_out.append(toks[:B])
                if step + 1 < so.num_step:
                    ops.step_advance(md.positions, md.seq_lens, md.slot_mapping, md.block_table, self.cfg.block_size, 1)
                    md.q_seq_lens = md.seq_lens
                    md.max_seq_len += 1
                    if md.omni is not None:      # the windows of the compressed layers move on with the sequence
                        nxt = self.omni.decode_metadata(md.seq_lens, md.omni["prompt_lens"], md.omni["block_table"])
                        md.omni = dict(md.omni, **nxt)
                    ids = toks
                continue
            # ---- MTP: verify the drafts, then draft again from the last accepted position
            fwd = toks.view(padded, tpr)
            u = None
            if 0.0 <= self.cfg.control_accept_rate <= 1.0:
                u = torch.rand(padded * (tpr - 1), device=self.device, generator=self.rng)
            out_tok, acc, last_idx, mtp_in = ops.mtp_verify(ids.view(padded, tpr), fwd, u, self.cfg.control_accept_rate)
            steps_out.append(out_tok[:B])
            drafts, h, cur = [], hidden, mtp_in.view(-1)
            for di, d in enumerate(self.drafters):
                h = d(cur, md, self.drafter_kv[di], h)
                dl = d.compute_logits(h[last_idx.long()])
                draft = ops.argmax(dl)
                drafts.append(draft)
                if di + 1 < len(self.drafters):
                    nxt = torch.roll(cur, -1)
                    nxt[last_idx.long()] = draft
                    cur = nxt
            draft_t = torch.stack(drafts, dim=1)                       # [padded, n_drafters]
            if draft_t.shape[1] < tpr - 1:
                draft_t = torch.nn.functional.pad(draft_t, (0, tpr - 1 - draft_t.shape[1]))
            spec_final = draft_t
            if step + 1 < so.num_step:
                adv = (acc + 1).int()
                ops.step_advance(md.positions, md.seq_lens, md.slot_mapping, md.block_table, self.cfg.block_size, tpr, adv)
                # visible kv tokens per q row: seq_len - tpr + j + 1
                base = (md.seq_lens - tpr).repeat_interleave(tpr)
                md.q_seq_lens = torch.where(base >= 0, base + torch.arange(1, tpr + 1, device=self.device, dtype=torch.int32).repeat(padded), torch.zeros_like(base)).int()
                md.max_seq_len += tpr
                last_tok = fwd.gather(1, acc.long().unsqueeze(1))
                ids = torch.cat([last_tok, draft_t], dim=1).reshape(-1)
        self._dummy_rounds(rounds - so.num_step)
        # ---- one host sync for the whole round
        if tpr == 1:
            stacked = torch.stack(steps_out, dim=0).tolist()           # [steps][B]
            sampled = [[[t] for t in row] for row in stacked]
            return ModelRunnerOutput([r.request_id for r in reqs], sampled, None)
        stacked = torch.stack(steps_out, dim=0).tolist()               # [steps][B][tpr]
        spec = spec_final[:B].tolist() if spec_final is not None else None
        return ModelRunnerOutput([r.request_id for r in reqs], stacked, spec)

    # ------------------------------------------------------------------ warm-up / dummy batches
    @torch.inference_mode()
    def execute_dummy_batch(self, num_tokens: int = 1) -> None:
        """An idle data-parallel rank still takes part in the step: it joins the agreement and runs as many rounds
        (main model + drafters, no live row) as the busiest rank, so that every expert-parallel exchange finds its
        peer (omni/adaptors/vllm/worker/npu_worker.py:285)."""
        padded = self._get_closest_gear(1) if self.graphs is not None else 1
        rounds = self._agree_ep_path(padded * self.tpr, 1, False)
        self._dummy_rounds(rounds)

    @torch.inference_mode()
    def profile_run(self) -> None:
        """One worst-case prefill to measure peak activation memory before sizing the KV cache."""
        n = min(self.cfg.max_num_batched_tokens, self.cfg.max_model_len - 1)
        cfg = self.model_cfg
        bs = self.cfg.block_size
        nblk = (n + bs - 1) // bs + 1
        self.initialize_kv_cache(nblk + 1)
        ids = torch.zeros(n, dtype=torch.int64, device=self.device)
        blocks = list(range(1, nblk + 1))
        md = AttnMetadata(True, torch.arange(n, device=self.device), self._to_dev(self._slots(blocks, 0, n), torch.int64),
                          self._to_dev([blocks], torch.int32), self._to_dev([n], torch.int32),
                          cu_q=self._to_dev([0, n], torch.int32), cu_k=self._to_dev([0, n], torch.int32),
                          query_lens=[n], context_lens=[0], max_q=n, max_k=n,
                          sample_indices=self._to_dev([n - 1], torch.int64))
        h = self.model(ids, md, self.kv_caches)
        self.model.compute_logits(h[md.sample_indices])
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        self.kv_caches, self.drafter_kv = [], []
