"""Request, sampling parameters and the scheduler <-> runner message types."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    seed: Optional[int] = None
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0


class RequestStatus(enum.IntEnum):
    WAITING = 0
    WAITING_FOR_REMOTE_KVS = 1
    RUNNING = 2
    PREEMPTED = 3
    FINISHED_STOPPED = 4
    FINISHED_LENGTH_CAPPED = 5
    FINISHED_ABORTED = 6
    FINISHED_IGNORED = 7

    @property
    def finished(self) -> bool:
        return self >= RequestStatus.FINISHED_STOPPED


FINISH_REASON = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH_CAPPED: "length",
                 RequestStatus.FINISHED_ABORTED: "abort", RequestStatus.FINISHED_IGNORED: "ignored"}


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list
    sampling: SamplingParams = field(default_factory=SamplingParams)
    arrival_time: float = field(default_factory=time.monotonic)
    priority: int = 0
    eos_token_id: Optional[int] = None
    # PD disaggregation: {"do_remote_prefill": bool, "do_remote_decode": bool, "remote_block_ids": [...],
    #  "remote_engine_id": ..., "remote_host": ..., "prefilled_token": int, "spec_token_ids": [...]}
    kv_transfer_params: Optional[dict] = None
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list = field(default_factory=list)
    spec_token_ids: list = field(default_factory=list)   # drafts to verify in the next step
    num_computed_tokens: int = 0
    num_cached_tokens: int = 0                           # prefix-cache hits at admission
    block_ids: list = field(default_factory=list)
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    num_preemptions: int = 0
    events: list = field(default_factory=list)           # (timestamp, action) timeline
    role: str = ""                                       # prefill / decode / mixed: names the engine in timeline lines

    @property
    def all_token_ids(self) -> list:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_tokens_with_spec(self) -> int:
        return self.num_tokens + len(self.spec_token_ids)

    @property
    def is_finished(self) -> bool:
        return self.status.finished

    def record(self, action: str) -> None:
        now = time.time()
        self.events.append((now, action))
        from ..utils import timeline
        if timeline.enabled():
            timeline.emit(action, self.request_id, role=self.role or None, ts=now)


@dataclass
class ScheduledRequest:
    request: Request
    num_scheduled_tokens: int      # tokens run through the model this step (prompt chunk, or 1 + drafts)
    is_prefill: bool
    spec_token_ids: list = field(default_factory=list)


@dataclass
class SchedulerOutput:
    scheduled: list                # list[ScheduledRequest]; all prefill or all decode
    is_prefill: bool
    num_step: int = 1              # model steps covered by this scheduling round (multi-step decode)
    total_tokens: int = 0
    finished_req_ids: set = field(default_factory=set)
    preempted_req_ids: list = field(default_factory=list)
    kv_connector_metadata: Any = None

    @property
    def empty(self) -> bool:
        return not self.scheduled


@dataclass
class ModelRunnerOutput:
    req_ids: list
    # sampled_token_ids[step][i] = accepted tokens of request i at that model step (>=1 with MTP)
    sampled_token_ids: list
    spec_token_ids: Optional[list] = None      # next drafts per request
    finished_sending: set = field(default_factory=set)
    finished_recving: set = field(default_factory=set)
    failed_recving: set = field(default_factory=set)     # remote KV never arrived: prefill locally instead
    step_time_s: float = 0.0


@dataclass
class RequestOutput:
    request_id: str
    new_token_ids: list
    finished: bool
    finish_reason: Optional[str] = None
    kv_transfer_params: Optional[dict] = None
    num_prompt_tokens: int = 0
    num_output_tokens: int = 0
