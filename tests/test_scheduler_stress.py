"""Randomised runs of the scheduler and the KV block manager against a deterministic stand-in for the model runner.

The stand-in makes the next token a pure function of every token before it, so whatever the scheduler does on the way
(chunked prefill, prefix-cache hits, preemption and recompute, multi-step rounds, accepted and rejected drafts, aborts)
a request's output must equal the function applied along its own sequence.  After every call the block accounting is
checked: reference counts equal the number of holders, free / cached / held blocks partition the pool, and a scheduled
request owns enough blocks for what it is about to write."""
import hashlib
import random

import pytest

from omni_infer_b200.engine.kv_manager import KVCacheManager
from omni_infer_b200.engine.request import ModelRunnerOutput, Request, RequestStatus, SamplingParams
from omni_infer_b200.engine.scheduler import Scheduler, SchedulerConfig

VOCAB = 50


def next_token(tokens) -> int:
    h = hashlib.blake2b(repr(list(tokens)).encode(), digest_size=4).digest()
    return int.from_bytes(h, "little") % VOCAB


def expected_output(prompt, max_tokens, stop=()):
    seq, out = list(prompt), []
    while len(out) < max_tokens:
        t = next_token(seq)
        seq.append(t)
        out.append(t)
        if t in stop:
            break
    return out


def check_blocks(sched: Scheduler, kv: KVCacheManager):
    holders = {}
    live = [r for r in sched.requests.values() if r.block_ids]
    for r in live:
        assert len(set(r.block_ids)) == len(r.block_ids), f"{r.request_id} holds a block twice"
        for b in r.block_ids:
            holders[b] = holders.get(b, 0) + 1
    first = 1
    for b in range(first, kv.num_blocks):
        assert kv.ref[b] == holders.get(b, 0), (b, kv.ref[b], holders.get(b, 0))
    free, cached, held = list(kv.free_blocks), set(kv.evictable), set(holders)
    assert len(free) == len(set(free)), "a block is on the free list twice"
    assert not (set(free) & cached) and not (set(free) & held) and not (cached & held)
    assert set(free) | cached | held == set(range(first, kv.num_blocks))
    assert 0 not in holders and kv.ref[0] == 0
    for b in cached:
        assert b in kv.block_hash and kv.hash_to_block.get(kv.block_hash[b]) == b
    for h, b in kv.hash_to_block.items():
        assert kv.block_hash.get(b) == h
    if hasattr(kv, "window_free"):                      # Omni-Attention: the pool of per-request windows
        held_w = [b for r in sched.requests.values() for b in (getattr(r, "omni_block_ids", None) or [])]
        assert len(held_w) == len(set(held_w)) and not (set(held_w) & set(kv.window_free))
        assert len(kv.window_free) == len(set(kv.window_free))
        assert set(held_w) | set(kv.window_free) == set(range(1, kv.num_window_blocks))
        n = kv.spec.blocks_per_request
        for r in sched.requests.values():
            w = getattr(r, "omni_block_ids", None) or []
            assert len(w) in (0, n) and (len(w) == n) == bool(r.block_ids), r.request_id
    # finished requests own nothing unless a hand-over is pending
    for r in sched.requests.values():
        if r.is_finished and r.request_id not in sched.pending_free:
            assert not r.block_ids, r.request_id


def fake_runner(so, rnd, num_spec):
    """What the model runner would return for this scheduler output."""
    reqs = [s.request for s in so.scheduled]
    ids = [r.request_id for r in reqs]
    if so.is_prefill:
        row = []
        for s in so.scheduled:
            r = s.request
            done = r.num_computed_tokens + s.num_scheduled_tokens >= r.num_tokens
            row.append([next_token(r.all_token_ids)] if done else [-1])
        spec = [[rnd.randrange(VOCAB) for _ in range(num_spec)] for _ in reqs] if num_spec else None
        return ModelRunnerOutput(ids, [row], spec)
    steps = []
    grown = {r.request_id: list(r.all_token_ids) for r in reqs}
    for _ in range(so.num_step):
        row = []
        for s in so.scheduled:
            seq = grown[s.request.request_id]
            accepted = rnd.randint(0, len(s.spec_token_ids)) if s.spec_token_ids else 0
            toks = []
            for _k in range(accepted + 1):
                t = next_token(seq)
                seq.append(t)
                toks.append(t)
            row.append(toks + [-1] * (1 + num_spec - len(toks)))
        steps.append(row)
    spec = [[rnd.randrange(VOCAB) for _ in range(num_spec)] for _ in reqs] if num_spec else None
    return ModelRunnerOutput(ids, steps, spec)


CASES = [
    dict(blocks=12, bs=4, seqs=4, budget=32, chunked=False, prefix=False, num_step=1, spec=0),
    dict(blocks=14, bs=4, seqs=6, budget=24, chunked=True, prefix=False, num_step=1, spec=0),
    dict(blocks=16, bs=4, seqs=5, budget=40, chunked=False, prefix=True, num_step=1, spec=0),
    dict(blocks=16, bs=4, seqs=4, budget=32, chunked=False, prefix=False, num_step=3, spec=0),
    dict(blocks=20, bs=4, seqs=4, budget=32, chunked=False, prefix=False, num_step=1, spec=2),
    dict(blocks=24, bs=4, seqs=5, budget=28, chunked=True, prefix=True, num_step=2, spec=1),
    dict(blocks=40, bs=8, seqs=8, budget=64, chunked=True, prefix=True, num_step=2, spec=3),
    dict(blocks=16, bs=4, seqs=4, budget=32, chunked=False, prefix=False, num_step=1, spec=0, omni_windows=3),
    dict(blocks=30, bs=4, seqs=6, budget=24, chunked=True, prefix=False, num_step=2, spec=0, omni_windows=2),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(f"{k}{v}" for k, v in c.items()))
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_traffic_keeps_outputs_and_block_accounting_right(case, seed):
    rnd = random.Random(1000 * seed + case["blocks"])
    if case.get("omni_windows"):
        # two pools: paged blocks plus a fixed window (1 sink + 3 recent blocks) per request; room for only a few windows
        from omni_infer_b200.accelerators.cache import OmniAttentionSpec, OmniKVCacheManager
        spec = OmniAttentionSpec(case["bs"], 1, 3)
        kv = OmniKVCacheManager(case["blocks"], case["bs"], spec, num_window_blocks=case["omni_windows"] * 4 + 1)
    else:
        kv = KVCacheManager(case["blocks"], case["bs"], enable_prefix_caching=case["prefix"])
    cfg = SchedulerConfig(max_num_seqs=case["seqs"], max_num_batched_tokens=case["budget"], max_model_len=64,
                          num_speculative_tokens=case["spec"], num_step=case["num_step"], enable_chunked_prefill=case["chunked"])
    sched = Scheduler(cfg, kv)
    shared = [rnd.randrange(VOCAB) for _ in range(3 * case["bs"])]        # a prefix several prompts share
    pending, all_reqs, aborted, outputs = [], {}, set(), {}
    for i in range(30):
        body = [rnd.randrange(VOCAB) for _ in range(rnd.randint(1, 18))]
        prompt = (shared[: rnd.choice([0, case["bs"], 2 * case["bs"], 3 * case["bs"]])] + body)[: case["budget"] if not case["chunked"] else 40]
        stop = (rnd.randrange(VOCAB),) if rnd.random() < 0.3 else ()
        req = Request(f"r{i}", prompt, SamplingParams(max_tokens=rnd.randint(1, 12), stop_token_ids=stop, ignore_eos=True))
        pending.append((rnd.randint(0, 60), req))
        all_reqs[req.request_id] = req
    pending.sort(key=lambda x: x[0])
    step = idle = 0
    while pending or sched.has_unfinished:
        while pending and pending[0][0] <= step:
            sched.add_request(pending.pop(0)[1])
        if rnd.random() < 0.05 and sched.requests:
            victim = rnd.choice(list(sched.requests))
            if not sched.requests[victim].is_finished:
                sched.abort_request(victim)
                aborted.add(victim)
        check_blocks(sched, kv)
        so = sched.schedule()
        check_blocks(sched, kv)
        # ---- what a step may look like
        kinds = {s.is_prefill for s in so.scheduled}
        assert len(kinds) <= 1 and (not so.scheduled or so.is_prefill == next(iter(kinds)))
        assert len(sched.running) <= cfg.max_num_seqs
        assert len({s.request.request_id for s in so.scheduled}) == len(so.scheduled)
        if so.is_prefill:      # within the budget, except a recompute that could never fit: that one runs alone
            total = sum(s.num_scheduled_tokens for s in so.scheduled)
            assert total <= cfg.max_num_batched_tokens or (len(so.scheduled) == 1 and not cfg.enable_chunked_prefill)
        look = (cfg.num_step - 1) * (1 + cfg.num_speculative_tokens) if not so.is_prefill else 0
        for s in so.scheduled:
            r = s.request
            assert r.status == RequestStatus.RUNNING and r in sched.running
            assert len(r.block_ids) * kv.block_size >= r.num_computed_tokens + s.num_scheduled_tokens + look, r.request_id
            if s.is_prefill:
                assert r.num_computed_tokens + s.num_scheduled_tokens <= r.num_tokens
                if not cfg.enable_chunked_prefill:
                    assert r.num_computed_tokens + s.num_scheduled_tokens == r.num_tokens
            else:
                assert r.num_computed_tokens == r.num_tokens - 1
        for rid in so.preempted_req_ids:
            assert all_reqs[rid].status == RequestStatus.PREEMPTED and not all_reqs[rid].block_ids
        if so.scheduled:
            idle = 0
            for ro in sched.update_from_output(so, fake_runner(so, rnd, cfg.num_speculative_tokens)):
                outputs.setdefault(ro.request_id, []).extend(ro.new_token_ids)
        elif sched.has_unfinished:
            idle += 1
            assert idle < 3, "requests are queued but nothing gets scheduled"
        check_blocks(sched, kv)
        step += 1
        assert step < 5000, "the scheduler makes no progress"
    # ---- the end state
    assert not sched.running and not sched.waiting
    assert kv.num_free_blocks == kv.num_blocks - 1
    finished = 0
    for rid, r in all_reqs.items():
        assert r.is_finished, rid
        if rid in aborted or r.status == RequestStatus.FINISHED_IGNORED:
            continue
        finished += 1
        want = expected_output(r.prompt_token_ids, min(r.sampling.max_tokens, cfg.max_model_len - len(r.prompt_token_ids)),
                               r.sampling.stop_token_ids)
        assert r.output_token_ids == want, (rid, r.num_preemptions)
        assert outputs.get(rid, []) == want, rid            # what was streamed is the output, once, in order
    assert finished >= 20
    if case["blocks"] <= 16:
        assert sched.stats["preemptions"] > 0 or case["prefix"]     # the small pools really were under pressure
    if case.get("omni_windows"):
        assert len(kv.window_free) == kv.num_window_blocks - 1


def test_a_preempted_request_longer_than_the_step_budget_is_not_stuck():
    """Without chunked prefill a preempted request recomputes prompt + generated tokens in one step.  When that exceeds
    the step's token budget it used to wait at the head of the queue for ever; it now runs in a step of its own."""
    kv = KVCacheManager(16, 4)
    cfg = SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=16, max_model_len=64)
    sched = Scheduler(cfg, kv)
    rnd = random.Random(0)
    long_req = Request("long", list(range(14)), SamplingParams(max_tokens=12, ignore_eos=True))
    sched.add_request(long_req)
    outputs = {}

    def step():
        so = sched.schedule()
        if so.scheduled:
            for ro in sched.update_from_output(so, fake_runner(so, rnd, 0)):
                outputs.setdefault(ro.request_id, []).extend(ro.new_token_ids)
        check_blocks(sched, kv)
        return so

    for _ in range(6):                                   # prefill + five decodes: 19 tokens, more than the budget of 16
        step()
    assert long_req.num_tokens > cfg.max_num_batched_tokens and not long_req.is_finished
    sched.running.remove(long_req)                       # what running out of blocks does to the last running request
    sched._preempt(long_req)
    other = Request("other", list(range(20, 26)), SamplingParams(max_tokens=3, ignore_eos=True))
    sched.add_request(other)
    so = step()
    assert [s.request.request_id for s in so.scheduled] == ["long"] and so.is_prefill     # alone, in an oversize step
    assert so.scheduled[0].num_scheduled_tokens == long_req.num_tokens - 1 > cfg.max_num_batched_tokens
    for _ in range(40):
        if not sched.has_unfinished:
            break
        step()
    assert long_req.output_token_ids == expected_output(long_req.prompt_token_ids, 12)
    assert other.output_token_ids == expected_output(other.prompt_token_ids, 3)
    # a fresh prompt that merely does not fit what is left of the current step still waits for the next one
    a = Request("a", list(range(10)), SamplingParams(max_tokens=1, ignore_eos=True))
    b = Request("b", list(range(30, 40)), SamplingParams(max_tokens=1, ignore_eos=True))
    sched.add_request(a)
    sched.add_request(b)
    so = sched.schedule()
    assert [s.request.request_id for s in so.scheduled] == ["a"]


@pytest.mark.parametrize("chunked", [False, True])
def test_a_request_that_outgrows_the_whole_pool_ends_instead_of_recomputing_for_ever(chunked):
    """Five usable blocks of four tokens; a request that wants 6 + 40 tokens can never hold them all.  It is ended with
    what it has generated (reason: length) at the point where even an empty pool would not do, its blocks are freed, the
    client hears about it, and the next request runs."""
    kv = KVCacheManager(6, 4)
    cfg = SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=16, max_model_len=256, enable_chunked_prefill=chunked)
    sched = Scheduler(cfg, kv)
    rnd = random.Random(0)
    big = Request("big", list(range(6)), SamplingParams(max_tokens=40, ignore_eos=True))
    small = Request("small", list(range(10, 13)), SamplingParams(max_tokens=2, ignore_eos=True))
    sched.add_request(big)
    seen = {}
    for i in range(60):
        if i == 3:
            sched.add_request(small)
        so = sched.schedule()
        out = fake_runner(so, rnd, 0) if so.scheduled else ModelRunnerOutput([], [[]])
        for ro in sched.update_from_output(so, out):
            seen.setdefault(ro.request_id, []).append(ro)
        check_blocks(sched, kv)
        if not sched.has_unfinished and i > 3:
            break
    assert big.status == RequestStatus.FINISHED_LENGTH_CAPPED and not big.block_ids
    assert 0 < len(big.output_token_ids) < 40 and big.num_tokens == 5 * 4 + 1      # the pool's 20 tokens + the last sample
    assert big.output_token_ids == expected_output(big.prompt_token_ids, 40)[: len(big.output_token_ids)]
    assert seen["big"][-1].finished and seen["big"][-1].finish_reason == "length"
    assert small.output_token_ids == expected_output(small.prompt_token_ids, 2)
    assert sched.stats.get("kv_capacity_stops") == 1 and kv.num_free_blocks == 5


def test_priority_policy_preempts_the_least_urgent_request():
    """With the priority policy the request that gives way when the KV pool runs out is the least urgent running one
    (largest priority value; the latest arrival among equals), not simply the last admitted, and it goes back into the
    queue at its place rather than ahead of more urgent waiting requests."""
    kv = KVCacheManager(10, 4)                          # 9 usable blocks
    cfg = SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=64, policy="priority")
    sched = Scheduler(cfg, kv)
    rnd = random.Random(0)
    # three requests of 8 prompt tokens (2 blocks each): urgent (0), background (5), normal (1) - admitted in that order
    reqs = {}
    for name, prio, t in (("urgent", 0, 1.0), ("background", 5, 2.0), ("normal", 1, 3.0)):
        r = Request(name, list(range(8)), SamplingParams(max_tokens=20, ignore_eos=True), priority=prio, arrival_time=t)
        reqs[name] = r
        sched.add_request(r)
    preempted_order = []
    for _ in range(40):
        so = sched.schedule()
        preempted_order += list(so.preempted_req_ids)
        if so.scheduled:
            sched.update_from_output(so, fake_runner(so, rnd, 0))
        check_blocks(sched, kv)
        if len(preempted_order) >= 1:
            break
    assert preempted_order[0] == "background"           # not "normal", which was admitted last
    # a more urgent request arrives while "background" waits: it is served first
    late = Request("late-urgent", list(range(8)), SamplingParams(max_tokens=2, ignore_eos=True), priority=0, arrival_time=9.0)
    sched.add_request(late)
    assert [r.request_id for r in sched.waiting] == ["late-urgent", "background"]
    done = {}
    for _ in range(400):
        if not sched.has_unfinished:
            break
        so = sched.schedule()
        if so.scheduled:
            for ro in sched.update_from_output(so, fake_runner(so, rnd, 0)):
                if ro.finished:
                    done[ro.request_id] = len(done)
        check_blocks(sched, kv)
    assert set(done) == {"urgent", "background", "normal", "late-urgent"}
    assert done["late-urgent"] < done["background"]
    for r in list(reqs.values()) + [late]:
        assert r.output_token_ids == expected_output(r.prompt_token_ids, r.sampling.max_tokens)


def test_the_table_of_finished_requests_is_bounded():
    """Finished requests stay in ``requests`` for callers that read an output after the last step, but only the latest
    ``KEEP_FINISHED`` of them: a server's table must not grow with every request it has ever served."""
    kv = KVCacheManager(16, 4)
    sched = Scheduler(SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=64), kv)
    sched.KEEP_FINISHED = 5
    rnd = random.Random(0)
    for i in range(20):
        sched.add_request(Request(f"r{i}", [1 + i, 2, 3], SamplingParams(max_tokens=2, ignore_eos=True)))
        if i == 7:
            sched.abort_request("r7")                     # dropped requests age out the same way
    for _ in range(60):
        if not sched.has_unfinished:
            break
        so = sched.schedule()
        sched.update_from_output(so, fake_runner(so, rnd, 0))
        check_blocks(sched, kv)
    assert not sched.has_unfinished and len(sched.requests) == 5 and "r19" in sched.requests and "r7" not in sched.requests
    assert kv.num_free_blocks == kv.num_blocks - 1
    # an id that has aged out (or merely finished) can be used again without touching the old record
    again = Request("r19", [9, 9], SamplingParams(max_tokens=1, ignore_eos=True))
    sched.add_request(again)
    for _ in range(10):
        if not sched.has_unfinished:
            break
        so = sched.schedule()
        sched.update_from_output(so, fake_runner(so, rnd, 0))
    assert sched.requests["r19"] is again and again.output_token_ids == expected_output([9, 9], 1)
