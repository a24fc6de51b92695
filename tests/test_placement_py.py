"""Python side of OmniPlacement on CPU: mapping/selector, router remap + activation histogram, a full dynamic
round on one rank, the offline pattern tool, and an engine run with redundant slots."""
import numpy as np
import pytest
import torch

from omni_infer_b200 import ops
from omni_infer_b200.accelerators.placement import ExpertMapping, OmniPlanner, base_pattern
from omni_infer_b200.accelerators.placement import pattern_tool


def test_expert_mapping_validation_and_selector():
    m = ExpertMapping(None, world=4, rank=2, layers=2, experts=8, redundant_per_rank=1)
    assert m.slots_per_rank == 3 and m.get_num_of_redundant_experts() == 4
    assert m.selector_dev[0].tolist() == [0, 1, 3, 4, 6, 7, 9, 10]
    assert m.is_expert_on_current_rank(0, 4) and not m.is_expert_on_current_rank(0, 0)
    assert m.update(0, 8, -1, 0)                       # replica of expert 0 on own rank (slot 2)
    assert m.selector_dev[0, 0].item() == 8 and m.get_redundant_count(0, 0) == 2
    bad = base_pattern(4, 2, 8)
    bad[0, 0, 0] = 0
    with pytest.raises(ValueError):
        ExpertMapping(bad, 4, 0, 2, 8)
    with pytest.raises(ValueError):
        ExpertMapping(np.ones((4, 2, 8), dtype=np.int32), 4, 0, 2, 8)
    m.close()


def test_router_remap_and_histogram():
    OmniPlanner.cleanup()
    pl = OmniPlanner(num_moe_layers=1, num_experts=8, max_redundant_per_rank=2, _new=True)
    logits = torch.randn(16, 8)
    ids, w = ops.router_topk(logits, 2, selector=pl.selector(0), counts=pl.activation_counts(0))
    ref_ids, _ = ops.router_topk_ref(logits, 2)
    assert torch.equal(ids, pl.plan(0, ref_ids))
    assert int(pl.sent_counts.sum()) == 32
    OmniPlanner.cleanup()


def test_dynamic_round_single_rank_engine():
    """World of 1 with redundant slots: the greedy balancer cannot move load between ranks, so a round is a no-op,
    but registration, collection and apply run end to end and the engine output does not change."""
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams

    OmniPlanner.cleanup()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]
    base = EngineCore(EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu"))
    for p in prompts:
        base.add_request(p, SamplingParams(max_tokens=6))
    want = base.run_until_done()
    eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu",
                                  placement_config={"max_redundant_per_rank": 2, "device": "cpu", "apply_interval": 2}))
    pl = eng.worker.runner.planner
    assert pl is not None and pl.slots_per_rank == 10
    for p in prompts:
        eng.add_request(p, SamplingParams(max_tokens=6))
    got = eng.run_until_done()
    assert [got[k] for k in sorted(got)] == [want[k] for k in sorted(want)]
    assert int(pl.sent_counts.sum()) > 0
    assert pl.run_round() >= 0
    pl.apply_pending()
    assert "max_over_mean_rank_load" in pl.load_stats()
    OmniPlanner.cleanup()


def test_pattern_tool(tmp_path):
    layers, experts, world = 3, 16, 4
    rng = np.random.default_rng(0)
    loads = rng.zipf(1.5, size=(layers, experts)).astype(np.float64)
    for i in range(2):
        np.savetxt(tmp_path / f"dump{i}.txt", loads / 2, fmt="%.1f")
    out = tmp_path / "pattern.npy"
    assert pattern_tool.main(["--dumps", str(tmp_path), "--world", str(world), "--redundant-per-rank", "2",
                              "--out", str(out)]) == 0
    pat = np.load(out)
    assert pat.shape == (world, layers, experts)
    pattern_tool.check_pattern(pat, 2)
    before = pattern_tool.analyse(base_pattern(world, layers, experts), loads)
    after = pattern_tool.analyse(pat, loads)
    assert after["max_over_mean_rank_load"] < before["max_over_mean_rank_load"]
    # the generated pattern loads into the mapping
    ExpertMapping(pat, world, 1, layers, experts, redundant_per_rank=2).close()
