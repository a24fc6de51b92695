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


def _write_dumps(folder, counts, parts=2):
    folder.mkdir(exist_ok=True)
    for i in range(parts):
        np.savetxt(folder / f"activation_rank0_{i}.txt", counts / parts, fmt="%d")


def test_pattern_tool_steps_from_logs_to_analysis(tmp_path, capsys):
    """logs -> CSV (mode and step filters, tiles, malformed lines), CSV -> patterns in both modes with a special-layer
    count, check + view, analysis table: each step reads the file the previous one wrote."""
    layers, world, per = 3, 4, 2
    log = tmp_path / "act.log"
    lines = []
    rng = np.random.default_rng(0)
    truth = np.zeros((layers, world * per))
    for step in range(10):
        for r in range(world):
            for l in range(layers):
                v = rng.integers(0, 300, per)
                if l == 1 and r == 0:
                    v[0] += 5000                      # layer 1: expert 0 is hot
                mode = "decode" if step % 2 else "prefill"
                lines.append(f"INFO xyz [dump activation] {mode} step {step} in rank {r} for layer {l} get {per} experts data: "
                             + "\t".join(map(str, v)))
                if mode == "decode" and 3 <= step <= 8:
                    truth[l, r * per:(r + 1) * per] += np.ceil(v / 128)
    lines.append("[dump activation] decode step 4 in rank 9 for layer 0 get 2 experts data: 1\t2")      # rank out of range
    lines.append("[dump activation] decode step 4 in rank 0 for layer 0 get 3 experts data: 1\t2\t3")   # wrong width
    lines.append("unrelated line")
    log.write_text("\n".join(lines) + "\n")
    csv_path = tmp_path / "counts.csv"
    assert pattern_tool.main(["logs-to-csv", "--inputs", str(log), "--input-mode", "log", "--layers", str(layers),
                              "--world-of-data", str(world), "--positions", str(world * per), "--collecting-mode", "decode",
                              "--step-range", "3:8", "--tile", "128", "--out", str(csv_path)]) == 0
    import json
    info = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert info["skipped_lines"] == 2 and info["layers"] == layers and info["columns"] == world * per
    got = pattern_tool.read_csv(str(csv_path))
    assert np.array_equal(got, truth)
    with pytest.raises(ValueError):
        pattern_tool.parse_step_range("9:3")

    outdir = tmp_path / "patterns"
    assert pattern_tool.main(["generate", "--csv", str(csv_path), "--outdir", str(outdir), "--world", str(world),
                              "--mode", "all", "--redundant-per-rank", "1", "--special-layers", "-1", "1"]) == 0
    names = sorted(p.name for p in outdir.iterdir())
    assert names == ["pattern_rearrange_1layers_4ranks.npy", "pattern_rearrange_alllayers_4ranks.npy",
                     "pattern_redundant_1layers_4ranks.npy", "pattern_redundant_alllayers_4ranks.npy"]
    base = base_pattern(world, layers, world * per)
    one = np.load(outdir / "pattern_redundant_1layers_4ranks.npy")
    assert one.shape == (world, layers, world * per)
    assert np.array_equal(one[:, 0], base[:, 0]) and np.array_equal(one[:, 2], base[:, 2])     # only the worst layer changed
    assert one[:, 1, 0].sum() >= 2                                                            # its hot expert is replicated
    re = np.load(outdir / "pattern_rearrange_alllayers_4ranks.npy")
    assert (re.sum(axis=0) == 1).all() and (re.sum(axis=2) == per).all()                      # a permutation per layer

    view = tmp_path / "view.txt"
    assert pattern_tool.main(["check", "--pattern", str(outdir / "pattern_redundant_1layers_4ranks.npy"),
                              "--redundant-per-rank", "1", "--view", str(view)]) == 0
    text = view.read_text()
    assert "layer 1:" in text and "0*" in text and "rank 3:" in text
    broken = one.copy()
    broken[:, 0, 3] = 0
    np.save(tmp_path / "broken.npy", broken)
    with pytest.raises(AssertionError):
        pattern_tool.main(["check", "--pattern", str(tmp_path / "broken.npy")])

    table = tmp_path / "analysis.csv"
    capsys.readouterr()
    assert pattern_tool.main(["analyse", "--csv", str(csv_path), "--patterns", *[str(outdir / n) for n in names],
                              "--out", str(table)]) == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["mean_max_over_mean"]
    assert summary["pattern_redundant_alllayers_4ranks"] < summary["base"]
    assert summary["pattern_rearrange_alllayers_4ranks"] <= summary["base"] + 1e-9
    import csv
    rows = list(csv.DictReader(open(table)))
    assert len(rows) == 5 * layers and {"deployment", "layer", "rank_0", "best", "max", "max_over_mean",
                                        "max_load_reduction"} <= set(rows[0])
    hot = [r for r in rows if r["deployment"] == "pattern_redundant_alllayers_4ranks" and r["layer"] == "1"][0]
    assert float(hot["max_load_reduction"]) > 0.3


def test_pattern_tool_pipeline_and_incremental_plan(tmp_path, capsys):
    import json
    layers, world, per, red = 2, 4, 2, 1
    slots = per + red
    counts = np.full((layers, world * per), 40.0)
    counts[0, 0] = 900
    dumps = tmp_path / "decode"
    _write_dumps(dumps, counts)
    work = tmp_path / "work"
    assert pattern_tool.main(["pipeline", "--inputs", str(dumps), "--world", str(world), "--redundant-per-rank", str(red),
                              "--workdir", str(work)]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["mean_max_over_mean"]["pattern_redundant_alllayers_4ranks"] < out["mean_max_over_mean"]["base"]
    for f in ("topk_id_count.csv", "load_analysis.csv", "pattern_redundant_alllayers_4ranks.npy",
              "pattern_redundant_alllayers_4ranks.view.txt"):
        assert (work / f).exists(), f

    # incremental plan from the base layout with per-position dumps taken under it
    cur = base_pattern(world, layers, world * per)
    np.save(tmp_path / "cur.npy", cur)
    placement = pattern_tool.pattern_to_placement(cur, slots)
    pos_counts = np.zeros_like(placement, dtype=np.float64)
    for l in range(layers):
        for p, e in enumerate(placement[l]):
            if e >= 0:
                pos_counts[l, p] = counts[l, e]
    pdumps = tmp_path / "pos"
    _write_dumps(pdumps, pos_counts, parts=1)
    plan_path = tmp_path / "plan.json"
    assert pattern_tool.main(["plan", "--current-pattern", str(tmp_path / "cur.npy"), "--dumps", str(pdumps), "--slots", str(slots),
                              "--diff-limit", "2", "--out", str(plan_path)]) == 0
    plan = json.loads(plan_path.read_text())
    ins = plan["instructions"]
    assert 1 <= len(ins) <= 2 and all(i["layer"] == 0 for i in ins)          # layer 1 is flat: nothing planned
    assert ins[0]["op"] == "add" and ins[0]["source_expert"] == 0 and ins[0]["wave"] == 1
    assert plan["ratio_after"][0] < plan["ratio_before"][0] - 0.1 and plan["ratio_after"][1] == plan["ratio_before"][1]
    # the library call agrees and rejects a bad placement
    ins2, ratios = pattern_tool.plan_instructions(placement, pos_counts, world, world * per, diff_limit=2)
    assert ins2 == ins and ratios.shape == (layers, 2)
    bad = placement.copy()
    bad[0, 0] = 1
    with pytest.raises(RuntimeError):
        pattern_tool.plan_instructions(bad, pos_counts, world, world * per)


def test_token_level_optimizers():
    """The six routing post-processors of the reference's ``optim`` package and their loader."""
    from omni_infer_b200.accelerators.placement import optim

    # 4 ranks x 3 slots, 8 experts; expert 0 also on rank 2, expert 5 also on rank 0
    pat = base_pattern(4, 1, 8)
    pat[2, 0, 0] = 1
    pat[0, 0, 5] = 1
    m = ExpertMapping(pat, world=4, rank=0, layers=1, experts=8, redundant_per_rank=1)
    place = m.placement()[0].tolist()
    pos0 = [p for p, e in enumerate(place) if e == 0]
    pos5 = [p for p, e in enumerate(place) if e == 5]
    assert len(pos0) == 2 and len(pos5) == 2
    ids = torch.tensor([[0, 5], [0, 3], [5, 0], [0, 7]])
    w = torch.full((4, 2), 0.5)

    # HEAT: own rank first, then own host, then the rank's offset
    for rank, want0 in ((0, pos0[0]), (2, pos0[1]), (3, pos0[1]), (1, pos0[0])):     # hosts of two ranks: {0,1}, {2,3}
        h = optim.HEATExpertsBalancer(m, rank=rank, ranks_per_host=2)
        _, out, _ = h.optimize(0, None, ids, w)
        assert out[0, 0].item() == want0, (rank, out.tolist())
        assert place[out[1, 1].item()] == 3                 # single-replica experts go to their only position
    far = optim.HEATExpertsBalancer(m, rank=1, ranks_per_host=1)     # no replica on its rank or host: offset 1 % 2
    assert far.optimize(0, None, ids, w)[1][0, 0].item() == pos0[1]
    assert optim.HEATExpertsBalancer(m, rank=1, ranks_per_host=1, global_offset=True).optimize(0, None, ids, w)[1][0, 0].item() == pos0[0]

    # Redundant2: replicas alternate with the token index
    r2 = optim.Redundant2ExpertsBalancer(m, rank=0)
    _, out, _ = r2.optimize(0, None, ids, w)
    assert [place[p] for p in out.flatten().tolist()] == ids.flatten().tolist()      # always a position of the same expert
    assert out[0, 0].item() != out[1, 0].item()             # tokens 0 and 1 hit different replicas of expert 0

    # ResDis: even deal without loads, all to the replica with room when the other rank is full
    rd = optim.ResDisExpertsBalancer(m)
    big = torch.zeros(40, 1, dtype=torch.long)
    _, out, _ = rd.optimize(0, None, big, torch.ones(40, 1))
    assert sorted(out.flatten().bincount(minlength=12)[pos0].tolist()) == [20, 20]
    loads = torch.tensor([1000.0, 10.0, 10.0, 10.0])         # rank 0 is far above the mean: no room there
    _, out, _ = rd.optimize(0, None, big, torch.ones(40, 1), cluster_status=loads)
    assert out.flatten().bincount(minlength=12)[pos0[1]].item() == 40
    capped = optim.ResDisExpertsBalancer(m, max_count=10).optimize(0, None, big, torch.ones(40, 1))[1]
    assert capped.flatten().bincount(minlength=12)[pos0[0]].item() == 35     # 5 + the 30 beyond the cap
    rnd = optim.ResDisExpertsBalancer(m, random=True, seed=1).optimize(0, None, big, torch.ones(40, 1))[1]
    assert set(rnd.flatten().tolist()) == set(pos0)

    # loader: the reference's "<module>.<Class>" names, keyword arguments, unknown names refused
    opts = optim.create_optimizers([{"ada_router_optimizer.AdaRouter": {"threshold": 0.5}},
                                    {"token_balance_optimizer.TokenBalance": {"capacity_factor": 1.0}},
                                    {"heat_optimizer.HEAT_ExpertsBalancer": {"ranks_per_host": 2}},
                                    {"ResDis_ExpertsBalancer": {"max_count": 16}}], mapping=m, rank=2, num_experts=8)
    assert [type(o).__name__ for o in opts] == ["AdaRouter", "TokenBalance", "HEATExpertsBalancer", "ResDisExpertsBalancer"]
    assert opts[2].rank == 2 and opts[1].E == 8
    w_in = torch.tensor([[0.9, 0.1], [0.5, 0.5], [0.6, 0.4], [0.8, 0.3]])
    _, i2, w2 = opts[0].optimize(0, None, ids, w_in)
    assert i2[0, 1].item() == -1 and abs(float(w2[0].sum()) - 1.0) < 1e-6     # AdaRouter dropped the weak choice, mass kept
    assert i2[1].tolist() == ids[1].tolist() and i2[3, 1].item() == -1
    _, i3, w3 = opts[1].optimize(0, None, i2, w2)                               # capacity 1 pair per expert at this size
    kept = i3[i3 >= 0]
    assert kept.bincount(minlength=8).max().item() == 1 and float(w3[i3 < 0].abs().sum()) == 0.0
    with pytest.raises(ValueError):
        optim.create_optimizers([{"NoSuchOptimizer": {}}])
    m.close()


def test_shipped_configuration_patterns_and_guideline(tmp_path):
    """The configuration file that ships with the package loads with the reference's keys, the base patterns are
    valid for their model shapes, and the commands of the guideline exist in the pattern tool."""
    import os
    import re
    import numpy as np
    import yaml
    from omni_infer_b200.accelerators.placement import OmniPlanner, pattern_tool
    from omni_infer_b200.models.config import tiny_deepseek_v3
    here = os.path.dirname(pattern_tool.__file__)
    cfg_path = os.path.join(here, "config.yaml")
    cfg = yaml.safe_load(open(cfg_path))
    assert {"pattern_path", "max_moe_layer_num", "enable_dynamic", "max_redundant_per_expert", "max_redundant_per_rank",
            "enable_dump", "dump_dir"} <= set(cfg)
    assert cfg["max_moe_layer_num"] == 58 and cfg["max_redundant_per_expert"] == 10 and cfg["max_redundant_per_rank"] == 1
    pl = OmniPlanner.from_config({"config_path": cfg_path}, tiny_deepseek_v3())
    try:
        assert pl.num_redundant_per_rank == 1 and pl.layers == 1 and not pl.enable_dynamic
    finally:
        OmniPlanner.cleanup()
    for name, (world, layers, experts) in {"DSV3_baseline_58_layers_8_ranks.npy": (8, 58, 256),
                                           "Qwen3_30B_A3B_baseline_48_layers_8_ranks.npy": (8, 48, 128)}.items():
        pat = np.load(os.path.join(here, "patterns", "base_patterns", name))
        assert pat.shape == (world, layers, experts) and set(np.unique(pat)) == {0, 1}
        assert (pat.sum(0) == 1).all() and (pat.sum(2) == experts // world).all()      # every expert once, ranks even
    guide = open(os.path.join(here, "Guideline.md")).read()
    for sub in re.findall(r"pattern_tool (\\w[\\w-]*)", guide) + re.findall(r"`([a-z-]+)`(?=[,)]| run)", guide):
        if sub in ("logs-to-csv", "generate", "check", "analyse", "plan", "pipeline"):
            with pytest.raises(SystemExit) as ei:
                pattern_tool.main([sub, "--help"])
            assert ei.value.code == 0
    for flag in re.findall(r"(--[a-z][a-z-]+)", guide):
        assert flag in open(pattern_tool.__file__).read(), flag
