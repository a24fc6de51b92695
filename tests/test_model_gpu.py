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


def test_small_deepseek_graph_vs_eager_and_mtp():
    prompts = _prompts(5, 40, 4096, seed=2)
    sp = SamplingParams(max_tokens=12)
    kw = dict(block_size=128, num_kv_blocks=32, max_model_len=1024, max_num_seqs=8,
              model_overrides={"num_nextn_predict_layers": 1})
    eager = LLM("small-deepseek", enforce_eager=True, **kw).generate(prompts, sp)
    graph = LLM("small-deepseek", **kw).generate(prompts, sp)
    assert _agreement(graph, eager) > 0.6       # random weights: near-tied logits flip under reordered reductions
    multi = LLM("small-deepseek", num_step=4, **kw).generate(prompts, sp)
    assert _agreement(multi, graph) > 0.6
    mtp = LLM("small-deepseek", num_speculative_tokens=1, **kw).generate(prompts, sp)
    assert _agreement(mtp, graph) > 0.6


def test_qwen_models_run():
    for name, over in (("qwen2-small", {}), ("qwen3-30b-a3b", {"num_hidden_layers": 2, "vocab_size": 4096})):
        llm = LLM(name, block_size=128, num_kv_blocks=16, max_model_len=512, max_num_seqs=4, model_overrides=over)
        outs = llm.generate(_prompts(3, 33, 4096, seed=3), SamplingParams(max_tokens=6))
        assert all(len(o) == 6 for o in outs)
