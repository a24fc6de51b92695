"""PD disaggregation on CPU: a prefill engine and a decode engine in one process, KV blocks pushed between their
paged caches, prefilled-token reuse, acknowledgement-driven block release, and host-side fault injection (dropped
and duplicated control messages, a transfer that never completes -> local-prefill fallback)."""
import time

import pytest
import torch

from omni_infer_b200.accelerators.pd import InProcessHub
from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
from omni_infer_b200.engine.request import SamplingParams


def _engine(role, name, **kw):
    cfg = EngineConfig(block_size=16, num_kv_blocks=48, max_model_len=160, device="cpu", seed=0,
                       kv_transfer_config={"kv_role": role, "engine_id": name, "endpoint": f"inproc://{name}",
                                           "sync_timeout_s": kw.pop("sync_timeout_s", 5.0), "retries": kw.pop("retries", 3),
                                           "retry_wait_s": kw.pop("retry_wait_s", 0.2)}, **kw)
    return EngineCore(cfg)


def _prompts(n=3, length=40, seed=4):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def _run_pd(P, D, prompts, max_tokens, deadline_s=30.0):
    # prefill instance: one token, KV kept
    for i, p in enumerate(prompts):
        P.add_request(p, SamplingParams(max_tokens=1), request_id=f"r{i}", kv_transfer_params={"do_remote_decode": True})
    handoff = {}
    while P.scheduler.has_unfinished:
        for out in P.step():
            if out.finished:
                handoff[out.request_id] = out.kv_transfer_params
    assert all(v and v["remote_block_ids"] for v in handoff.values())
    for i, p in enumerate(prompts):
        D.add_request(p, SamplingParams(max_tokens=max_tokens), request_id=f"r{i}", kv_transfer_params=dict(handoff[f"r{i}"]))
    outs = {}
    t0 = time.time()
    while D.has_unfinished and time.time() - t0 < deadline_s:
        for out in D.step():
            outs.setdefault(out.request_id, []).extend(out.new_token_ids)
        P.step()              # lets the producer observe finished_sending and free its blocks
        time.sleep(0.001)
    return outs


@pytest.fixture(autouse=True)
def _reset_hub():
    InProcessHub.reset()
    yield
    InProcessHub.reset()


def _mixed_reference(prompts, max_tokens):
    E = EngineCore(EngineConfig(block_size=16, num_kv_blocks=48, max_model_len=160, device="cpu", seed=0))
    ids = [E.add_request(p, SamplingParams(max_tokens=max_tokens)) for p in prompts]
    outs = E.run_until_done()
    return [outs[i] for i in ids]


def test_pd_matches_single_instance_and_frees_producer_blocks():
    prompts = _prompts()
    want = _mixed_reference(prompts, 8)
    P, D = _engine("kv_producer", "p0"), _engine("kv_consumer", "d0")
    free_before = P.kv.num_free_blocks
    outs = _run_pd(P, D, prompts, 8)
    assert [outs[f"r{i}"] for i in range(len(prompts))] == want
    for _ in range(20):
        P.step()
    assert P.kv.num_free_blocks == free_before and not P.scheduler.pending_free
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 0


def test_dropped_push_request_is_retried_and_duplicate_acks_ignored():
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 5)
    P, D = _engine("kv_producer", "p1"), _engine("kv_consumer", "d1")
    InProcessHub.drop_next = 1
    InProcessHub.duplicate_acks = True
    outs = _run_pd(P, D, prompts, 5)
    assert [outs[f"r{i}"] for i in range(2)] == want


def test_transfer_that_never_completes_falls_back_to_local_prefill():
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 5)
    P = _engine("kv_producer", "p2")
    D = _engine("kv_consumer", "d2", sync_timeout_s=0.6, retries=1, retry_wait_s=0.2)
    InProcessHub.drop_next = 100           # the producer never hears about the requests
    outs = _run_pd(P, D, prompts, 5)
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 2
    assert [outs[f"r{i}"] for i in range(2)] == want
