"""Whole-model checks on the GPU: the small MLA+MoE model through the engine (CUDA kernels, CUDA graphs)
against the fp32 oracle running on the same weights."""
import pytest
import torch

from omni_infer_b200.engine.engine_core import LLM
from omni_infer_b200.engine.request import SamplingParams
from omni_infer_b200.models.reference_fp32 import ReferenceDeepseek

pytestmark = pytest.mark.gpu


def _prompts(n, length, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _agreement(a, b):
    tot = sum(len(x) for x in a)
    same = 0
    for x, y in zip(a, b):
        for i, (u, v) in enumerate(zip(x, y)):
            if u != v:
                break
            same += 1
    return same / tot


@pytest.mark.parametrize("quant", ["none", "fp8_block"])
def test_small_deepseek_logits_vs_oracle(quant):
    """Prefill logits of the CUDA path track the fp32 oracle on the same (de-quantised) weights."""
    llm = LLM("small-deepseek", block_size=128, num_kv_blocks=16, max_model_len=1024, enforce_eager=True,
              model_overrides={"quantization": quant})
    runner = llm.engine.worker.runner
    sd = {k: v for k, v in runner.model.state_dict().items()}
    ref = ReferenceDeepseek(llm.engine.model_cfg, sd)
    prompt = _prompts(1, 48, 4096, seed=1)[0]
    want = ref.logits(prompt)[-1]
    eng = llm.engine
    eng.add_request(prompt, SamplingParams(max_tokens=1))
    so = eng.scheduler.schedule()
    ids, md = runner._prepare_prefill(so)
    with torch.inference_mode():
        h = runner.model(ids, md, runner.kv_caches)
        got = runner.model.compute_logits(h[md.sample_indices])[0].float().cpu()
    cos = torch.nn.functional.cosine_similarity(got, want, dim=0).item()
    assert cos > (0.98 if quant == "fp8_block" else 0.995), cos


def _assert_near_oracle_argmax(ref, prompts, outs, tol_sigma, what):
    """Teacher-forced check of generated tokens: at every step the chosen token's fp32-oracle logit must lie within
    ``tol_sigma`` standard deviations (of that step's logits) of the oracle's maximum.  With 4096 random-weight logits
    the maximum sits about 3.7 sigma out, so a token picked from wrong state (a missed KV write, a stale graph input,
    a mis-ordered draft) fails this by a wide margin, while a flip between two near-tied candidates passes."""
    worst = 0.0
    for p, o in zip(prompts, outs):
        lg = ref.logits(list(p) + list(o[:-1]))
        for i, tok in enumerate(o):
            row = lg[len(p) - 1 + i]
            gap = (row.max() - row[tok]).item() / row.std().item()
            worst = max(worst, gap)
            assert gap <= tol_sigma, f"{what}: step {i} token {tok} is {gap:.2f} sigma below the oracle's best"
    return worst


def _oracle_of(llm):
    from omni_infer_b200.models.reference_fp32 import reference_for
    return reference_for(llm.engine.model_cfg, dict(llm.engine.worker.runner.model.state_dict()))


def test_small_deepseek_graph_multistep_and_mtp_tokens_vs_oracle():
    """Every decode path (eager, CUDA graph, 4 steps per schedule, MTP speculative) is held to the fp32 oracle at
    every generated position, not only to the first token: 12 steps cross the KV writes, graph replays with growing
    context, and draft acceptance."""
    prompts = _prompts(5, 40, 4096, seed=2)
    sp = SamplingParams(max_tokens=12)
    kw = dict(block_size=128, num_kv_blocks=32, max_model_len=1024, max_num_seqs=8,
              model_overrides={"num_nextn_predict_layers": 1})
    ref = None
    for what, extra in (("eager", {"enforce_eager": True}), ("graph", {}), ("multi-step", {"num_step": 4}),
                        ("mtp", {"num_speculative_tokens": 1})):
        llm = LLM("small-deepseek", **extra, **kw)
        ref = ref or _oracle_of(llm)           # same seed, same weights in every variant
        outs = llm.generate(prompts, sp)
        assert all(len(o) == 12 for o in outs)
        _assert_near_oracle_argmax(ref, prompts, outs, 0.75, what)
        # first tokens come from the prefill, where bf16 noise is smallest: they match the oracle's argmax outright
        firsts = [int(ref.logits(p)[-1].argmax()) for p in prompts]
        assert sum(o[0] == f for o, f in zip(outs, firsts)) >= 4, what


def test_fp8_block_decode_tokens_vs_oracle():
    prompts = _prompts(3, 40, 4096, seed=4)
    llm = LLM("small-deepseek", block_size=128, num_kv_blocks=32, max_model_len=1024, max_num_seqs=8,
              model_overrides={"quantization": "fp8_block"})
    outs = llm.generate(prompts, SamplingParams(max_tokens=10))
    _assert_near_oracle_argmax(_oracle_of(llm), prompts, outs, 1.0, "fp8 graph")   # oracle runs on the de-quantised weights


@pytest.mark.parametrize("name,over", [("qwen2-small", {}),
                                       ("qwen3-30b-a3b", {"num_hidden_layers": 2, "vocab_size": 4096})])
def test_qwen_models_tokens_vs_oracle(name, over):
    """Dense GQA (biased qkv) and the GQA MoE with q/k norm (128 experts, top-8) against their fp32 oracle."""
    prompts = _prompts(3, 33, 4096, seed=3)
    for what, extra in (("eager", {"enforce_eager": True}), ("graph", {})):
        llm = LLM(name, block_size=128, num_kv_blocks=16, max_model_len=512, max_num_seqs=4, model_overrides=over, **extra)
        outs = llm.generate(prompts, SamplingParams(max_tokens=6))
        assert all(len(o) == 6 for o in outs)
        _assert_near_oracle_argmax(_oracle_of(llm), prompts, outs, 0.75, f"{name} {what}")
