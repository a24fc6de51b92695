"""Prefill-first hybrid scheduler with multi-step decode, speculative tokens and PD states.

Behaviour follows the reference's NpuHybridScheduler (omni/adaptors/vllm/worker/npu_schedule.py:87-559)
and the engine patches it relies on:

* a step is all-prefill or all-decode; waiting requests are admitted FCFS while the token budget and
  ``max_num_seqs`` allow; without chunked prefill a prompt is scheduled whole or not at all, and a
  prompt that exceeds the remaining budget stops admission (chunk_prefill_enable.patch);
* only when no prefill was scheduled do running requests decode: one new token each plus their draft
  tokens; on KV exhaustion the tail of ``running`` is preempted;
* one scheduling round may cover ``num_step`` model steps (multi_step.patch): KV slots for the
  look-ahead ``(num_step-1) * (1+num_spec)`` are allocated up front and the per-step outputs are
  reconciled in ``update_from_output``;
* requests whose KV arrives from a prefill instance wait in WAITING_FOR_REMOTE_KVS, then start with
  ``num_computed_tokens = num_tokens - 1`` (scheduler_kv_cache_manager_partial_kv_transfer.patch); on
  the prefill side a finished request hands its block ids to the connector and its blocks are freed
  only when the connector reports ``finished_sending``;
* speculative ids are seeded with zeros after a remote-KV arrival (mtp.patch).
"""
from __future__ import annotations

import os
import threading
from collections import deque
from dataclasses import dataclass
from typing import Optional

from .kv_manager import KVCacheManager
from .request import (FINISH_REASON, ModelRunnerOutput, Request, RequestOutput, RequestStatus, ScheduledRequest,
                      SchedulerOutput)


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 4096
    num_speculative_tokens: int = 0
    num_step: int = 1                       # multi-step decode
    async_schedule: bool = False
    enable_chunked_prefill: bool = os.environ.get("FORCE_ENABLE_CHUNK_PREFILL", "0") == "1"
    policy: str = "fcfs"                    # fcfs | priority


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, kv: KVCacheManager, connector=None):
        self.cfg, self.kv, self.connector = cfg, kv, connector
        self.waiting: deque = deque()
        self.running: list = []
        self.requests: dict = {}
        self.finished_req_ids: set = set()
        self._finished_order: deque = deque() # finished requests still listed in ``requests``, oldest first
        self.pending_free: dict = {}          # prefill side: blocks kept until the decode side pulled them
        self.finished_recving: set = set()
        self.pull_kv_lock = threading.Lock()  # serialises the fast-path KV pull with schedule()
        self._aborting: dict = {}             # dropped while their KV transfer ran: finished when it has concluded
        self._capacity_stopped: list = []     # (request, new tokens) ended inside schedule(): reported with the next outputs
        self.stats = {"preemptions": 0, "scheduled_prefill_tokens": 0, "scheduled_decode_tokens": 0, "steps": 0}

    KEEP_FINISHED = 1024

    # ------------------------------------------------------------------ intake
    def add_request(self, req: Request) -> None:
        self.requests[req.request_id] = req
        req.record("Enter scheduler waiting queue")
        if self.cfg.policy == "priority":
            items = sorted(list(self.waiting) + [req], key=lambda r: (r.priority, r.arrival_time))
            self.waiting = deque(items)
        else:
            self.waiting.append(req)

    def abort_request(self, request_id: str) -> None:
        req = self.requests.get(request_id)
        if req is None or req.is_finished or request_id in self._aborting:
            return
        if (req.status == RequestStatus.WAITING_FOR_REMOTE_KVS and req.block_ids and self.connector is not None
                and self.connector.abandon(request_id)):
            # A producer may be writing into these blocks right now.  Freeing them here would hand them to another
            # request while the copy still lands in them: the request ends when the transfer has been cancelled (it
            # then shows up as failed) or has completed.
            self._aborting[request_id] = req
            return
        self._finish(req, RequestStatus.FINISHED_ABORTED)
        if req in self.running:
            self.running.remove(req)
        try:
            self.waiting.remove(req)
        except ValueError:
            pass

    @property
    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_running(self) -> int:
        return len(self.running)

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)

    # ------------------------------------------------------------------ fast path (decode instance)
    def try_pull_kv_fast_path(self, req: Request) -> bool:
        """Called from the request-intake thread: allocate the KV slots of a remote-prefilled request
        and start the transfer at once instead of waiting for the next schedule() round
        (patch_support_fast_path_pull_kv.patch)."""
        if self.connector is None or not (req.kv_transfer_params or {}).get("do_remote_prefill"):
            return False
        with self.pull_kv_lock:
            n_ext, is_async = self.connector.get_num_new_matched_tokens(req, 0)
            if not is_async or self.kv.allocate_slots(req, n_ext) is None:
                return False
            req.status = RequestStatus.WAITING_FOR_REMOTE_KVS
            req.record("Start to pull kv (fast path)")
            self.connector.update_state_after_alloc(req, n_ext)
            self.connector.kick(self.connector.build_connector_meta())
            return True

    # ------------------------------------------------------------------ schedule
    def schedule(self) -> SchedulerOutput:
        with self.pull_kv_lock:
            return self._schedule()

    def _schedule(self) -> SchedulerOutput:
        cfg = self.cfg
        self.stats["steps"] += 1
        budget = cfg.max_num_batched_tokens
        scheduled: list = []
        preempted: list = []

        # -- requests whose remote KV has landed become runnable
        if self.finished_recving:
            for req in list(self.waiting):
                if req.status == RequestStatus.WAITING_FOR_REMOTE_KVS and req.request_id in self.finished_recving:
                    self.finished_recving.discard(req.request_id)
                    if self._aborting.pop(req.request_id, None) is not None:
                        self.waiting.remove(req)          # dropped meanwhile: the copy is over, the blocks can go
                        self._finish(req, RequestStatus.FINISHED_ABORTED)
                        continue
                    params = req.kv_transfer_params or {}
                    if params.get("prefilled_token") is not None and not req.output_token_ids:
                        # reuse the prefill instance's first token; it counts like any sampled token, so it can end the
                        # request (token cap of one, end-of-sequence, a stop id) before anything is decoded here
                        first: list = []
                        self._append(req, [int(params["prefilled_token"])], first)
                        if req.is_finished:
                            self.waiting.remove(req)
                            self.kv.free(req)
                            self._capacity_stopped.append((req, first))
                            continue
                        req._emit_prefilled = True
                    req.num_computed_tokens = req.num_tokens - 1
                    if cfg.num_speculative_tokens:
                        req.spec_token_ids = list(params.get("spec_token_ids") or [0] * cfg.num_speculative_tokens)
                    req.status = RequestStatus.RUNNING
                    req.record("Finish to pull kv")
                    self.waiting.remove(req)
                    self.running.append(req)

        # -- 0. partially prefilled running requests (chunked prefill) go on first: they are older than anything
        # waiting, and admitting newcomers ahead of them can take the blocks they need to ever finish.  When the
        # pool is exhausted the last running request is preempted, as in the decode phase.
        if cfg.enable_chunked_prefill:
            idx = 0
            while idx < len(self.running) and budget > 0:
                req = self.running[idx]
                rem = req.num_tokens - req.num_computed_tokens
                if rem <= 1:
                    idx += 1
                    continue
                n = min(rem, budget)
                ok = False
                while True:
                    if self.kv.allocate_slots(req, n) is not None:
                        ok = True
                        break
                    vi, victim = self._pop_victim()
                    if vi < idx:
                        idx -= 1
                    if victim is req and self._can_never_fit(req, n):
                        self._give_up(req)
                        break
                    self._preempt(victim)
                    preempted.append(victim.request_id)
                    if victim is req:
                        break
                if not ok:
                    break
                scheduled.append(ScheduledRequest(req, n, True))
                budget -= n
                idx += 1
            scheduled = [s for s in scheduled if s.request in self.running]

        # -- 1. admit waiting requests (prefill); not in a step that had to preempt (the victim heads the queue and
        # would come straight back)
        skipped: list = []
        while (self.waiting and budget > 0 and not preempted
               and len(self.running) + len([s for s in scheduled if s.request not in self.running]) < cfg.max_num_seqs):
            req = self.waiting[0]
            if req.status == RequestStatus.WAITING_FOR_REMOTE_KVS:
                skipped.append(self.waiting.popleft())
                continue
            params = req.kv_transfer_params or {}
            if self.connector is not None and params.get("do_remote_prefill") and req.num_computed_tokens == 0:
                n_ext, is_async = self.connector.get_num_new_matched_tokens(req, 0)
                if is_async:
                    if self.kv.allocate_slots(req, n_ext) is None:
                        break
                    req.status = RequestStatus.WAITING_FOR_REMOTE_KVS
                    req.record("Start to pull kv")
                    self.connector.update_state_after_alloc(req, n_ext)
                    skipped.append(self.waiting.popleft())
                    continue
            if req.num_prompt_tokens >= cfg.max_model_len or \
                    self.kv.blocks_needed(req.num_prompt_tokens + 1) > self.kv.num_blocks - 1:
                self.waiting.popleft()
                self._finish(req, RequestStatus.FINISHED_IGNORED)
                self._capacity_stopped.append((req, []))     # nobody else would tell the client: reported with the next outputs
                continue
            computed_blocks, n_cached = ([], 0)
            if req.num_computed_tokens == 0 and not req.block_ids:
                computed_blocks, n_cached = self.kv.get_computed_blocks(req)
            start = max(req.num_computed_tokens, n_cached)
            num_new = req.num_tokens - start
            if num_new > budget:
                if cfg.enable_chunked_prefill:
                    num_new = budget
                elif num_new > cfg.max_num_batched_tokens and not scheduled:
                    # It would not fit an empty step either (a preempted request recomputes its prompt plus what it
                    # has generated, which may exceed a budget its prompt alone respected): waiting cannot help and it
                    # would block the queue for ever.  It runs alone in a step of its own size.
                    pass
                else:
                    break          # the prompt does not fit this step: stop admitting
            if req.num_computed_tokens == 0 and n_cached:
                req.num_computed_tokens = n_cached
                req.num_cached_tokens = n_cached
            if self.kv.allocate_slots(req, num_new, computed_blocks) is None:
                if req.num_cached_tokens and not req.block_ids:
                    req.num_computed_tokens = 0     # the prefix references were handed back: start over next time
                    req.num_cached_tokens = 0
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            req.record("Prefill scheduled")
            scheduled.append(ScheduledRequest(req, num_new, True))
            budget -= num_new
        for r in reversed(skipped):
            self.waiting.appendleft(r)

        if scheduled:
            for s in scheduled:
                if s.request not in self.running:
                    self.running.append(s.request)
            total = sum(s.num_scheduled_tokens for s in scheduled)
            self.stats["scheduled_prefill_tokens"] += total
            return self._finalize(SchedulerOutput(scheduled, True, 1, total, preempted_req_ids=preempted))

        # -- 2. decode: only when no prefill was scheduled
        num_step = max(1, cfg.num_step)
        per_step = 1 + cfg.num_speculative_tokens
        lookahead = (num_step - 1) * per_step
        idx = 0
        while idx < len(self.running):
            req = self.running[idx]
            if req.num_computed_tokens < req.num_tokens - 1:
                idx += 1          # still prefilling (chunked) - handled above
                continue
            n = 1 + len(req.spec_token_ids)
            ok = False
            while True:
                if self.kv.allocate_slots(req, n, lookahead=lookahead) is not None:
                    ok = True
                    break
                # out of blocks: preempt the lowest-priority (last) running request
                vi, victim = self._pop_victim()
                if vi < idx:
                    idx -= 1
                if victim is req and self._can_never_fit(req, n + lookahead):
                    self._give_up(req)
                    break
                self._preempt(victim)
                preempted.append(victim.request_id)
                if victim is req:
                    break
            if not ok:
                break
            scheduled.append(ScheduledRequest(req, n, False, list(req.spec_token_ids)))
            idx += 1
        scheduled = [s for s in scheduled if s.request in self.running]
        total = sum(s.num_scheduled_tokens for s in scheduled)
        self.stats["scheduled_decode_tokens"] += total * num_step
        return self._finalize(SchedulerOutput(scheduled, False, num_step, total, preempted_req_ids=preempted))

    def _finalize(self, out: SchedulerOutput) -> SchedulerOutput:
        out.finished_req_ids = self.finished_req_ids
        self.finished_req_ids = set()
        if self.connector is not None:
            out.kv_connector_metadata = self.connector.build_connector_meta()
        return out

    def _pop_victim(self):
        """(index, request) of the running request that gives way when the KV pool is exhausted: the last one admitted,
        or with the priority policy the one of lowest priority (largest value, latest arrival among equals), as in the
        reference's scheduler (omni/adaptors/vllm/worker/npu_schedule.py:111-359)."""
        i = len(self.running) - 1
        if self.cfg.policy == "priority":
            i = max(range(len(self.running)), key=lambda k: (self.running[k].priority, self.running[k].arrival_time))
        return i, self.running.pop(i)

    def _can_never_fit(self, req: Request, num_new_tokens: int) -> bool:
        """The request wants more blocks than the whole pool has: preempting it would only bring it back to the same
        point after a recompute, for ever."""
        return self.kv.blocks_needed(req.num_computed_tokens + num_new_tokens) > self.kv.num_blocks - 1

    def _give_up(self, req: Request) -> None:
        """Ends a request that has outgrown the KV pool (it keeps what it has generated; reason: length)."""
        self.kv.free(req)
        self._finish(req, RequestStatus.FINISHED_LENGTH_CAPPED)
        self.stats["kv_capacity_stops"] = self.stats.get("kv_capacity_stops", 0) + 1
        self._capacity_stopped.append((req, []))

    def _preempt(self, req: Request) -> None:
        self.kv.free(req)
        req.status = RequestStatus.PREEMPTED
        req.num_computed_tokens = 0
        req.spec_token_ids = []
        req.num_preemptions += 1
        self.stats["preemptions"] += 1
        if self.cfg.policy == "priority":      # back into its place by priority, not ahead of more urgent requests
            self.waiting = deque(sorted(list(self.waiting) + [req], key=lambda r: (r.priority, r.arrival_time)))
        else:
            self.waiting.appendleft(req)

    # ------------------------------------------------------------------ results
    def update_from_output(self, sched: SchedulerOutput, out: ModelRunnerOutput) -> list:
        """Apply the runner's per-step token lists; returns one RequestOutput per request that progressed."""
        results: list = []
        if out.finished_recving:
            self.finished_recving |= set(out.finished_recving)
        for rid in getattr(out, "failed_recving", None) or ():
            # the remote KV never arrived: give the blocks back and prefill the prompt on this instance
            req = self.requests.get(rid)
            if req is not None and self._aborting.pop(rid, None) is not None:
                try:
                    self.waiting.remove(req)
                except ValueError:
                    pass
                self._finish(req, RequestStatus.FINISHED_ABORTED)
                continue
            if req is not None and req.status == RequestStatus.WAITING_FOR_REMOTE_KVS:
                self.kv.free(req)
                req.status = RequestStatus.WAITING
                req.num_computed_tokens = 0
                req.record("KV transfer failed: local prefill")
                self.stats["kv_fallbacks"] = self.stats.get("kv_fallbacks", 0) + 1
        for rid in out.finished_sending or ():
            req = self.pending_free.pop(rid, None)
            if req is not None:
                self.kv.free(req)          # safe when already freed
        for req, toks in self._capacity_stopped:
            results.append(RequestOutput(req.request_id, list(toks), True, FINISH_REASON.get(req.status), None,
                                         req.num_prompt_tokens, len(req.output_token_ids)))
        self._capacity_stopped = []
        idx_of = {rid: i for i, rid in enumerate(out.req_ids)}
        for s in sched.scheduled:
            req = s.request
            i = idx_of.get(req.request_id)
            if i is None or req.is_finished:
                continue
            new_tokens: list = []
            if getattr(req, "_emit_prefilled", False):
                new_tokens.append(req.output_token_ids[0])
                req._emit_prefilled = False
            if s.is_prefill:
                req.num_computed_tokens += s.num_scheduled_tokens
                if req.num_computed_tokens >= req.num_tokens:      # every known token has run: the sample is new
                    toks = [t for t in out.sampled_token_ids[0][i] if t >= 0]
                    self._append(req, toks[:1], new_tokens)
                    self.kv.cache_full_blocks(req)
            else:
                for step in range(len(out.sampled_token_ids)):
                    if req.is_finished:
                        break
                    toks = [t for t in out.sampled_token_ids[step][i] if t >= 0]
                    if not toks:
                        continue
                    req.num_computed_tokens += len(toks)
                    self._append(req, toks, new_tokens)
            if out.spec_token_ids is not None and not req.is_finished:
                req.spec_token_ids = list(out.spec_token_ids[i])
            kvp = None
            if req.is_finished:
                if req in self.running:
                    self.running.remove(req)
                kvp = self._free_or_hand_over(req)
            if new_tokens or req.is_finished:
                results.append(RequestOutput(req.request_id, new_tokens, req.is_finished,
                                             FINISH_REASON.get(req.status), kvp, req.num_prompt_tokens,
                                             len(req.output_token_ids)))
        return results

    def _append(self, req: Request, toks: list, sink: list) -> None:
        import time as _t

        sp = req.sampling
        for t in toks:
            req.output_token_ids.append(int(t))
            sink.append(int(t))
            if req.first_token_time is None:
                req.first_token_time = _t.monotonic()
                req.record("First token sampled")
            n_out = len(req.output_token_ids)
            if not sp.ignore_eos and req.eos_token_id is not None and t == req.eos_token_id:
                self._finish(req, RequestStatus.FINISHED_STOPPED)
            elif t in sp.stop_token_ids:
                self._finish(req, RequestStatus.FINISHED_STOPPED)
            elif n_out >= sp.max_tokens or req.num_tokens >= self.cfg.max_model_len:
                self._finish(req, RequestStatus.FINISHED_LENGTH_CAPPED)
            if req.is_finished:
                break

    def _finish(self, req: Request, status: RequestStatus) -> None:
        import time as _t

        req.status = status
        req.finish_time = _t.monotonic()
        req.record("Finish request")
        self.finished_req_ids.add(req.request_id)
        # finished requests stay readable for a while (callers look their outputs up after the last step), but not for
        # ever: a server lives for millions of requests
        self._finished_order.append(req)
        while len(self._finished_order) > self.KEEP_FINISHED:
            old = self._finished_order.popleft()
            if self.requests.get(old.request_id) is old:
                del self.requests[old.request_id]
        if status in (RequestStatus.FINISHED_ABORTED, RequestStatus.FINISHED_IGNORED):
            self.kv.free(req)

    def _free_or_hand_over(self, req: Request) -> Optional[dict]:
        """Prefill instance: a length-capped request keeps its blocks until the decode side has pulled them."""
        if self.connector is not None:
            delay, params = self.connector.request_finished(req, self.kv.get_block_ids(req)[0])
            if delay:
                self.pending_free[req.request_id] = req
                return params
            self.kv.free(req)
            return params
        self.kv.free(req)
        return None
