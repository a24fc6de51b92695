"""End-to-end on CPU: the engine (scheduler + paged latent cache + absorbed decode + fused-layout ops)
must reproduce the naive fp32 oracle token for token (tiny DeepSeek-V3-style MLA+MoE, 4 prompts of 32
tokens, 16 greedy tokens)."""
import pytest
import torch

from omni_infer_b200.engine.engine_core import LLM, EngineConfig, EngineCore
from omni_infer_b200.engine.request import SamplingParams
from omni_infer_b200.models.reference_fp32 import ReferenceDeepseek


def _prompts(n=4, length=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def _oracle(llm, prompts, n):
    ref = ReferenceDeepseek(llm.engine.model_cfg, llm.engine.worker.runner.model.state_dict())
    return [ref.greedy(p, n) for p in prompts]


def test_tiny_deepseek_token_exact():
    llm = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu")
    prompts = _prompts()
    outs = llm.generate(prompts, SamplingParams(max_tokens=16))
    assert outs == _oracle(llm, prompts, 16)


def test_multi_step_and_chunked_prefill_match():
    prompts = _prompts(3, 40, seed=1)
    base = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu")
    want = base.generate(prompts, SamplingParams(max_tokens=12))
    multi = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu", num_step=4)
    assert multi.generate(prompts, SamplingParams(max_tokens=12)) == want
    chunk = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu",
                enable_chunked_prefill=True, max_num_batched_tokens=24)
    assert chunk.generate(prompts, SamplingParams(max_tokens=12)) == want
    asyn = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu",
               async_schedule=True)
    assert asyn.generate(prompts, SamplingParams(max_tokens=12)) == want


def test_prefix_caching_and_preemption_match():
    prompts = _prompts(2, 48, seed=2)
    prompts.append(prompts[0][:32] + [5, 6, 7, 8])       # shares two full blocks with prompt 0
    base = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu")
    want = base.generate(prompts, SamplingParams(max_tokens=10))
    pc = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu",
             enable_prefix_caching=True, max_num_seqs=2)
    assert pc.generate(prompts, SamplingParams(max_tokens=10)) == want
    assert any(r.num_cached_tokens > 0 for r in pc.engine.scheduler.requests.values())
    # 10 usable blocks: the three prompts fit (9 blocks), growth forces a preemption and a recompute
    tight = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=11, max_model_len=128, device="cpu")
    assert tight.generate(prompts, SamplingParams(max_tokens=10)) == want
    assert tight.engine.scheduler.stats["preemptions"] > 0


def test_mtp_greedy_equivalence():
    """Speculative decoding with the MTP drafter never changes greedy output, whatever is accepted."""
    prompts = _prompts(3, 24, seed=3)
    over = {"num_nextn_predict_layers": 1}
    base = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu",
               model_overrides=over)
    want = base.generate(prompts, SamplingParams(max_tokens=14))
    mtp = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu",
              model_overrides=over, num_speculative_tokens=1)
    assert mtp.generate(prompts, SamplingParams(max_tokens=14)) == want
    mtp2 = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu",
               model_overrides=over, num_speculative_tokens=1, num_step=3)
    assert mtp2.generate(prompts, SamplingParams(max_tokens=14)) == want


def test_sampling_penalties_change_greedy_output():
    """A strong repetition penalty forbids tokens of the prompt and earlier outputs; presence / frequency penalties act on
    output tokens only.  Reference semantics: omni/models/common/layers/sampler.py:143-200."""
    import torch

    from omni_infer_b200.engine.engine_core import LLM
    from omni_infer_b200.engine.request import SamplingParams
    from omni_infer_b200.ops.sampling import apply_penalties_ref

    llm = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu", seed=0)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 1024, (24,), generator=g).tolist()
    plain = llm.generate([prompt], SamplingParams(max_tokens=12))[0]
    pen = llm.generate([prompt], SamplingParams(max_tokens=12, repetition_penalty=1e6))[0]
    assert len(set(pen)) == len(pen) and not (set(pen) & set(prompt))
    assert plain != pen or len(set(plain)) == len(plain)
    # reference arithmetic on a hand-made row
    logits = torch.tensor([[2.0, -1.0, 0.5, 3.0]])
    hist = torch.tensor([[0, 1, 3, 3, -1]], dtype=torch.int32)
    out = apply_penalties_ref(logits, hist, torch.tensor([2]), torch.tensor([2.0]), torch.tensor([0.5]), torch.tensor([0.25]))
    assert torch.allclose(out, torch.tensor([[1.0, -2.0, 0.5, 3.0 / 2 - 0.5 * 2 - 0.25]]))


@pytest.mark.parametrize("name,over", [("tiny-qwen3-moe", {}),
                                       ("qwen2-small", {"dtype": "float32", "hidden_size": 256, "intermediate_size": 512,
                                                        "head_dim": 32, "vocab_size": 1024})])
def test_qwen_models_match_their_fp32_oracle(name, over):
    """GQA models (dense with biased qkv; MoE with q/k norm and renormalised softmax routing) through the engine
    give exactly the oracle's greedy tokens on CPU."""
    from omni_infer_b200.models.reference_fp32 import reference_for
    llm = LLM(name, block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu", model_overrides=over)
    ref = reference_for(llm.engine.model_cfg, dict(llm.engine.worker.runner.model.state_dict()))
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (21,), generator=g).tolist() for _ in range(2)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=6))
    for p, o in zip(prompts, outs):
        assert o == ref.greedy(p, 6)


COMBOS = [
    dict(num_kv_blocks=12, enable_prefix_caching=True, enable_chunked_prefill=True, max_num_batched_tokens=24),
    dict(num_kv_blocks=12, num_step=3, enable_prefix_caching=True),
    dict(num_kv_blocks=14, num_speculative_tokens=1, num_step=2, mtp=True),
    dict(num_kv_blocks=14, num_speculative_tokens=1, enable_chunked_prefill=True, max_num_batched_tokens=20, mtp=True),
    dict(num_kv_blocks=13, async_schedule=True, num_step=2),
    dict(num_kv_blocks=13, num_speculative_tokens=1, num_step=2, enable_prefix_caching=True, async_schedule=True, mtp=True),
]


COMBOS += [dict(c, model="tiny-qwen3-moe") for c in COMBOS if not c.get("mtp")]


@pytest.mark.parametrize("combo", COMBOS, ids=lambda c: "-".join(f"{k}={v}" for k, v in c.items()))
def test_feature_combinations_under_memory_pressure_match_the_plain_engine(combo):
    """Features that each pass alone, together and with a KV pool small enough to force preemption and recompute:
    prefix cache + chunked prefill, multi-step, MTP drafts, asynchronous scheduling.  Greedy output must not change."""
    combo = dict(combo)
    model = combo.pop("model", "tiny-deepseek-v3")
    over = {"num_nextn_predict_layers": 1} if combo.pop("mtp", False) else {}
    g = torch.Generator().manual_seed(9)
    shared = torch.randint(0, 1024, (32,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 1024, (int(n),), generator=g).tolist() for n in (3, 9, 17)]
    prompts += [torch.randint(0, 1024, (int(n),), generator=g).tolist() for n in (21, 40)]
    base = LLM(model, block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu", model_overrides=over)
    want = base.generate(prompts, SamplingParams(max_tokens=18))
    llm = LLM(model, block_size=16, max_model_len=128, device="cpu", max_num_seqs=4, model_overrides=over, **combo)
    got = llm.generate(prompts, SamplingParams(max_tokens=18))
    assert got == want
    st = llm.engine.scheduler.stats
    assert st["preemptions"] > 0, st                     # the pool really was too small
    assert llm.engine.kv.num_free_blocks == combo["num_kv_blocks"] - 1


def test_priority_scheduling_serves_urgent_requests_first():
    """``scheduling_policy="priority"``: with room for one sequence at a time, requests finish in priority order however
    they arrived, and the tokens are those of the plain engine."""
    prompts = _prompts(3, 20, seed=5)
    base = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu")
    want = base.generate(prompts, SamplingParams(max_tokens=6))
    eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu", max_num_seqs=1,
                                  scheduling_policy="priority"))
    ids = [eng.add_request(p, SamplingParams(max_tokens=6), priority=pr) for p, pr in zip(prompts, (2, 0, 1))]
    order, outs = [], {}
    while eng.has_unfinished:
        for r in eng.step():
            outs.setdefault(r.request_id, []).extend(r.new_token_ids)
            if r.finished:
                order.append(r.request_id)
    assert order == [ids[1], ids[2], ids[0]]
    assert [outs[i] for i in ids] == want


@pytest.mark.parametrize("seed,kw,mtp", [
    (0, dict(num_kv_blocks=14, enable_prefix_caching=True, enable_chunked_prefill=True, max_num_batched_tokens=32), False),
    (1, dict(num_kv_blocks=16, num_step=3, scheduling_policy="priority"), False),
    (2, dict(num_kv_blocks=18, num_speculative_tokens=1, num_step=2, enable_prefix_caching=True), True),
    (3, dict(num_kv_blocks=16, async_schedule=True, enable_chunked_prefill=True, max_num_batched_tokens=24), False),
])
def test_random_arrivals_through_the_whole_engine(seed, kw, mtp):
    """Requests of random lengths arriving at random steps (some with a shared prefix, some with priorities) through
    scheduler, block manager, input preparation and the model under a small KV pool: every request's tokens equal what
    it gets when it is served alone by a plain engine."""
    import random
    rnd = random.Random(seed)
    over = {"num_nextn_predict_layers": 1} if mtp else {}
    g = torch.Generator().manual_seed(100 + seed)
    shared = torch.randint(0, 1024, (32,), generator=g).tolist()
    jobs = []
    for i in range(10):
        body = torch.randint(0, 1024, (rnd.randint(1, 40),), generator=g).tolist()
        prompt = (shared[: rnd.choice([0, 16, 32])] + body)[:60]
        jobs.append((rnd.randint(0, 25), prompt, rnd.randint(1, 14), rnd.randint(0, 2)))
    base = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu", model_overrides=over)
    want = [base.generate([p], SamplingParams(max_tokens=n))[0] for _, p, n, _ in jobs]
    eng = EngineCore(EngineConfig(block_size=16, max_model_len=128, device="cpu", max_num_seqs=4, model_overrides=over, **kw))
    pending = sorted(range(len(jobs)), key=lambda i: jobs[i][0])
    ids, outs, step = {}, {}, 0
    while pending or eng.has_unfinished:
        while pending and jobs[pending[0]][0] <= step:
            i = pending.pop(0)
            ids[i] = eng.add_request(jobs[i][1], SamplingParams(max_tokens=jobs[i][2]), priority=jobs[i][3])
        for r in eng.step():
            outs.setdefault(r.request_id, []).extend(r.new_token_ids)
        step += 1
        assert step < 3000
    assert [outs[ids[i]] for i in range(len(jobs))] == want
    assert eng.kv.num_free_blocks == kw["num_kv_blocks"] - 1


def test_abort_while_a_round_is_executing_under_async_scheduling():
    """With asynchronous scheduling a round runs on the worker thread while the caller may drop requests.  Dropping a
    request of the executing round used to free its blocks under the runner's feet; it now takes effect once the round's
    results are in.  The other requests are unaffected and nothing leaks."""
    prompts = _prompts(3, 30, seed=7)
    base = LLM("tiny-deepseek-v3", block_size=16, num_kv_blocks=64, max_model_len=128, device="cpu")
    want = base.generate(prompts, SamplingParams(max_tokens=10))
    for drop_at in range(1, 8):
        eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu", async_schedule=True,
                                      enable_chunked_prefill=True, max_num_batched_tokens=24))
        ids = [eng.add_request(p, SamplingParams(max_tokens=10)) for p in prompts]
        outs, step = {}, 0
        while eng.has_unfinished:
            if step == drop_at:
                eng.abort(ids[1])                         # a round is in flight at this point
            for r in eng.step():
                outs.setdefault(r.request_id, []).extend(r.new_token_ids)
            step += 1
            assert step < 500
        assert outs[ids[0]] == want[0] and outs[ids[2]] == want[2]
        assert outs.get(ids[1], []) == want[1][:len(outs.get(ids[1], []))]
        assert eng.scheduler.requests[ids[1]].status.name == "FINISHED_ABORTED"
        assert eng.kv.num_free_blocks == 31
