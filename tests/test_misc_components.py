"""Pangu parsers, mock model modes, profiler patches, typed config, platform plugin, topology tool."""
import json
import os
import sys
import types

import pytest
import torch

from omni_infer_b200.models.pangu import PanguReasoningParser, PanguToolParser


def test_pangu_reasoning_parser():
    p = PanguReasoningParser()
    assert p.extract_reasoning_content("[unused16]think[unused17]answer") == ("think", "answer")
    assert p.extract_reasoning_content("think more[unused17]final") == ("think more", "final")
    assert p.extract_reasoning_content("plain") == (None, "plain")
    assert p.extract_reasoning_content("[unused16]unfinished") == ("unfinished", None)
    prev, seen = "", {"reasoning_content": "", "content": ""}
    for d in ["[unus", "ed16]th", "ink", "[unused17]", "ans", "wer"]:
        m = p.extract_reasoning_content_streaming(prev, d)
        prev += d
        for k, v in (m or {}).items():
            seen[k] += v
    assert seen["content"] == "answer" and "ink" in seen["reasoning_content"]


def test_pangu_tool_parser():
    p = PanguToolParser()
    r = p.extract_tool_calls('Sure.[unused11]get_weather|{"city": "Paris", "unit": "c"}[unused12]')
    assert r.tools_called and r.content == "Sure." and r.tool_calls[0].name == "get_weather"
    assert json.loads(r.tool_calls[0].arguments) == {"city": "Paris", "unit": "c"}
    r2 = p.extract_tool_calls('[unused11][{"name": "a", "arguments": {"x": 1}}, {"name": "b", "arguments": {}}][unused12]')
    assert [c.name for c in r2.tool_calls] == ["a", "b"]
    assert not p.extract_tool_calls("no tools here").tools_called
    assert not p.extract_tool_calls("[unused11]broken|{not json[unused12]").tools_called
    prev, calls, text = "", [], ""
    for d in ["Hi ", "[unused11]f|{", '"a": 1}', "[unused12]", " done"]:
        m = p.extract_tool_calls_streaming(prev, d)
        prev += d
        if m and "tool_calls" in m:
            calls += m["tool_calls"]
        elif m:
            text += m["content"]
    assert len(calls) == 1 and calls[0]["function"]["name"] == "f" and "Hi" in text


def test_mock_model_random_capture_replay(tmp_path, monkeypatch):
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    from omni_infer_b200.models import mock, registry

    monkeypatch.setenv("MOCK_CAPTURE_DIR", str(tmp_path))
    prompts = [[1, 2, 3, 4], [9, 8, 7]]
    real = EngineCore(EngineConfig(block_size=16, num_kv_blocks=16, max_model_len=64, device="cpu"))
    ids = [real.add_request(p, SamplingParams(max_tokens=5)) for p in prompts]
    outs = real.run_until_done()
    mock.capture_outputs(prompts, [outs[i] for i in ids], step_ms=1.0)
    store = mock.ReplayStore(tmp_path / "capture.jsonl")
    assert store.next_token(prompts[0])[0] == outs[ids[0]][0]
    assert store.next_token(prompts[0] + outs[ids[0]][:2])[0] == outs[ids[0]][2]
    # random mode through the registry switch
    monkeypatch.setenv("RANDOM_MODE", "1")
    monkeypatch.setenv("KV_CACHE_MODE", "1")
    registry._REGISTRY.clear()
    try:
        eng = EngineCore(EngineConfig(block_size=16, num_kv_blocks=16, max_model_len=64, device="cpu"))
        assert type(eng.worker.runner.model).__name__.startswith("Mock")
        rid = eng.add_request([5, 6, 7], SamplingParams(max_tokens=4))
        assert len(eng.run_until_done()[rid]) == 4
        assert float(eng.worker.runner.kv_caches[0].abs().sum()) > 0
    finally:
        registry._REGISTRY.clear()


def test_profiler_patches(tmp_path):
    from omni_infer_b200.utils import profiler_patches as pp

    mod = types.ModuleType("omni_dummy_target")

    class K:
        def work(self, x, request_id=None):
            return x * 2

    mod.K = K
    mod.free = lambda x: x + 1
    sys.modules["omni_dummy_target"] = mod
    events = []
    pp.MARKER_CALLBACKS["enter"] = lambda a, k: events.append(("enter", k.get("request_id")))
    pp.MARKER_CALLBACKS["leave"] = lambda a, k, r: events.append(("leave", r))
    yml = tmp_path / "names.yml"
    yml.write_text("- {target: 'omni_dummy_target:K.work', type: marker, entry: enter, exit: leave}\n"
                   "- {target: 'omni_dummy_target.free', type: timer}\n- {target: 'nope.missing', type: timer}\n")
    done = pp.apply_patches(str(yml))
    assert done == ["omni_dummy_target:K.work", "omni_dummy_target.free"]
    assert mod.K().work(3, request_id="r1") == 6 and events == [("enter", "r1"), ("leave", 6)]
    assert mod.free(1) == 2 and len(pp.TIMINGS["omni_dummy_target.free"]) == 1


def test_config_sources_and_platform(tmp_path, monkeypatch):
    from omni_infer_b200 import envs
    from omni_infer_b200.adaptors.vllm.platform import B200Platform, ConfigUpdater, register
    from omni_infer_b200.config import AdditionalConfig, load_model_extra_config
    from omni_infer_b200.engine.engine_core import EngineConfig

    f = tmp_path / "extra.json"
    f.write_text(json.dumps({"model_parallel_config": {"dense_mlp_tp_size": 4, "dp_size": 8},
                             "operator_optimizition_config": {"moe_dispatch_combine": False, "gmm_nz": True,
                                                              "decode_gear_list": [64], "unknown_key": 1}}))
    cfg = load_model_extra_config(str(f))
    assert cfg.parall_config.dense_mlp_tp_size == 4 and cfg.operator_opt_config.decode_gear_list == [64]
    add = AdditionalConfig.from_json('{"graph_model_compile_config": {"level": 1, "decode_gear_list": [32], "use_ge_graph_cached": true},'
                                     ' "async_schedule": true, "multi_step": 4, "enable_omni_attn": true}')
    assert add.graph_model_compile_config.decode_gear_list == [32] and add.multi_step == 4 and add.async_schedule
    ec = EngineConfig(max_num_seqs=16)
    ConfigUpdater.update_engine_config(ec, {"graph_model_compile_config": {"level": 0}, "multi_step": 2}, str(f))
    assert ec.enforce_eager and ec.num_step == 2 and ec.decode_gear_list == [64] and ec.ep_backend == "nccl"
    monkeypatch.setenv("NO_GPU_MOCK", "1")
    assert register() == "omni_infer_b200.adaptors.vllm.platform.B200Platform"
    assert B200Platform.get_attn_backend_cls(True).endswith("MLAAttention")
    assert envs.NO_GPU_MOCK is True
    monkeypatch.setenv("OMNI_EP_WAIT_MS", "7")
    assert envs.OMNI_EP_WAIT_MS == 7
    with pytest.raises(AttributeError):
        envs.NOT_A_VARIABLE


def test_topology_tool(tmp_path):
    from omni_infer_b200.accelerators.pd import topology as T

    t = T.generate(4, 4)
    assert len(t.by_role("prefill")) == 4 and t.by_role("decode")[0].gpus == [4]
    t.save(str(tmp_path / "topo.json"))
    t2 = T.Topology.load(str(tmp_path / "topo.json"))
    assert t2.instances[5].control_endpoint == "tcp://127.0.0.1:5669"
    a, b = T.generate(1, 0), T.generate(0, 1)
    assert len(T.merge(a, b).instances) == 2
    with pytest.raises(ValueError):
        T.merge(a, a)
    # command line with the reference tool's option names
    d1, d2 = tmp_path / "t1", tmp_path / "t2"
    assert T.main(["--mode", "gen", "--prefill-server-list", "0,1", "2,3", "--decode-server-list", "4,5,6,7", "--save-dir", str(d1)]) == 0
    g = T.Topology.load(str(d1 / "global_topology.json"))
    assert [i.gpus for i in g.instances] == [[0, 1], [2, 3], [4, 5, 6, 7]] and g.instances[2].role == "decode"
    assert (d1 / "local_prefill-1.json").exists()
    assert T.main(["--mode", "merge", "--local-ranktable-list", str(d1 / "local_prefill-0.json"), str(d1 / "local_decode-0.json"),
                   "--save-dir", str(d2)]) == 0
    assert [i.name for i in T.Topology.load(str(d2 / "global_topology.json")).instances] == ["prefill-0", "decode-0"]
    with pytest.raises(SystemExit):
        T.main(["--mode", "gen", "--prefill-server-list", "0,1", "2", "--save-dir", str(d1)])      # unequal TP sizes
    with pytest.raises(SystemExit):
        T.main(["--mode", "gen", "--prefill-server-list", "0", "--decode-server-list", "0", "--save-dir", str(d1)])   # GPU used twice


def test_kv_manager_failed_allocation_hands_prefix_references_back():
    """A request that hits the prefix cache but then finds no room for the rest of its prompt must leave the block
    manager as it found it: cached blocks evictable again, no reference held, no block id on the request."""
    from omni_infer_b200.engine.kv_manager import KVCacheManager
    from omni_infer_b200.engine.request import Request

    kv = KVCacheManager(num_blocks=6, block_size=4, enable_prefix_caching=True)      # block 0 is the null block
    first = Request("a", list(range(10)))
    assert kv.allocate_slots(first, 10) is not None and len(first.block_ids) == 3
    first.num_computed_tokens = 10
    kv.cache_full_blocks(first)
    cached = first.block_ids[:2]
    kv.free(first)
    assert kv.num_free_blocks == 5 and all(kv.ref[b] == 0 for b in cached)

    # the same 8-token prefix, then a tail that needs 6 more blocks than there are
    second = Request("b", list(range(8)) + list(range(100, 120)))
    blocks, n_cached = kv.get_computed_blocks(second)
    assert blocks == cached and n_cached == 8
    second.num_computed_tokens = n_cached
    free_before = kv.num_free_blocks
    assert kv.allocate_slots(second, second.num_tokens - n_cached, blocks) is None
    assert second.block_ids == [] and kv.num_free_blocks == free_before
    assert all(kv.ref[b] == 0 for b in cached) and all(b in kv.evictable for b in cached)

    # and a request that fits still finds the cached prefix and takes it
    third = Request("c", list(range(8)) + [200, 201])
    blocks3, n3 = kv.get_computed_blocks(third)
    assert blocks3 == cached
    third.num_computed_tokens = n3
    assert kv.allocate_slots(third, third.num_tokens - n3, blocks3) is not None
    assert third.block_ids[:2] == cached and all(kv.ref[b] == 1 for b in cached)


def test_state_dir_round_trip_and_fingerprint(tmp_path):
    import numpy as np
    from omni_infer_b200.engine.state_dir import StateDir

    fp = {"model": "m", "world": 2, "block_size": 128}
    st = StateDir(str(tmp_path), rank=1, fp=fp)
    assert st.load() == {} and st.get("num_kv_blocks") is None and st.get_array("placement_ema") is None
    st.save(num_kv_blocks=321, graph_buckets=[1, 2, 4])
    st.save(placement_ema=np.arange(6, dtype=np.float64).reshape(2, 3))          # merges with what is there
    again = StateDir(str(tmp_path), rank=1, fp=dict(fp))
    assert again.get("num_kv_blocks") == 321 and again.get("graph_buckets") == [1, 2, 4]
    assert np.array_equal(again.get_array("placement_ema"), np.arange(6.0).reshape(2, 3))
    assert StateDir(str(tmp_path), rank=0, fp=fp).load() == {}                      # per rank
    assert StateDir(str(tmp_path), rank=1, fp={**fp, "block_size": 64}).load() == {}   # another configuration: ignored
    (tmp_path / "state_rank1.json").write_text("{ not json")
    assert StateDir(str(tmp_path), rank=1, fp=fp).load() == {}                      # unreadable: start cold
    assert not [f for f in os.listdir(tmp_path) if f.startswith(".tmp_")]          # no temporary file left behind


def test_engine_restart_reuses_block_count_placement_and_load_history(tmp_path):
    """First run: serves requests, runs a placement round (which builds the balancer's load history) and saves its
    state.  Second run with the same configuration starts from the saved block count, placement and history.  A run
    with another configuration starts cold."""
    import numpy as np
    from omni_infer_b200.accelerators.placement import OmniPlanner
    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams

    def make(**kw):
        OmniPlanner.cleanup()
        cfg = dict(block_size=16, num_kv_blocks=0, max_model_len=128, device="cpu", state_dir=str(tmp_path),
                   placement_config={"max_redundant_per_rank": 2, "device": "cpu"})
        cfg.update(kw)
        return EngineCore(EngineConfig(**cfg))

    first = make(num_kv_blocks=40)
    assert first.state.get("num_kv_blocks") == 40 and first.state.get("graph_buckets") == []
    pl = first.planner
    g = torch.Generator().manual_seed(0)
    first.add_request(torch.randint(0, 1024, (20,), generator=g).tolist(), SamplingParams(max_tokens=4))
    first.run_until_done()
    assert pl.run_round() >= 0
    first.save_state()
    saved_pos, saved_ema = first.state.get_array("placement_positions"), first.state.get_array("placement_ema")
    assert saved_pos.shape == saved_ema.shape == (pl.layers, pl.num_positions) and saved_ema.sum() > 0
    assert first.state.get_array("placement_pattern").shape == (pl.world, pl.layers, pl.experts)

    second = make()                                  # no block count given: taken from the state directory
    assert second.kv.num_blocks == 40
    assert np.array_equal(second.planner.mapping.placement(), saved_pos)
    second.planner.run_round()                       # builds the balancer, which takes the saved history first
    assert second.planner.pending_ema is None
    blended = second.planner.export_state()["placement_ema"]
    # nothing was routed in the second run, so its first round blends the restored history with zeros (keep = 0.6)
    assert np.allclose(blended, 0.6 * saved_ema)

    # the history follows the experts when a rank's slots come back in another order
    pl2 = second.planner
    perm = saved_pos.copy()
    perm[:, [0, 1]] = perm[:, [1, 0]]
    marked = np.zeros_like(saved_ema)
    marked[:, 0], marked[:, 1] = 7.0, 9.0            # saved under the permuted order: slot 0 held expert 1
    pl2.pending_ema = (perm, marked)
    pl2._restore_ema()
    now = pl2.export_state()["placement_ema"]
    assert np.all(now[:, 0] == 9.0) and np.all(now[:, 1] == 7.0)

    cold = make(block_size=32, num_kv_blocks=24)     # another block size: the saved state does not apply
    assert cold.kv.num_blocks == 24 and cold.state.get_array("placement_ema") is None
    OmniPlanner.cleanup()


def test_rope_scaling_variants():
    import math
    from omni_infer_b200.ops.basic import rope_cos_sin_table
    D, N, base = 64, 64, 10000.0
    plain = rope_cos_sin_table(D, N, base)
    inv = 1.0 / (base ** (torch.arange(0, D // 2, dtype=torch.float64) * 2 / D))
    assert torch.allclose(plain[:, :D // 2], torch.outer(torch.arange(N, dtype=torch.float64), inv).cos().float(), atol=1e-6)
    lin = rope_cos_sin_table(D, N, base, {"type": "linear", "factor": 4.0})
    assert torch.allclose(lin[4 * 3], plain[3], atol=1e-5)                       # position 12 of the stretched table = position 3
    l3 = rope_cos_sin_table(D, N, base, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                         "original_max_position_embeddings": 64})
    wavelen = 2 * math.pi / inv
    fast, slow = int((wavelen < 64 / 4.0).nonzero().max()), int((wavelen > 64 / 1.0).nonzero().min())
    assert torch.allclose(l3[:, fast], plain[:, fast], atol=1e-6)               # short wavelengths untouched
    assert torch.allclose(l3[8 * 5, slow], plain[5, slow], atol=1e-5)           # long ones slowed down by the factor
    mid = (fast + slow) // 2
    ang_mid = torch.acos(l3[1, mid].double().clamp(-1, 1))
    assert inv[mid] / 8.0 - 1e-9 <= ang_mid <= inv[mid] + 1e-9                  # the band between is interpolated
    dyn_short = rope_cos_sin_table(D, 32, base, {"type": "dynamic", "factor": 2.0, "original_max_position_embeddings": 32})
    assert torch.equal(dyn_short, rope_cos_sin_table(D, 32, base))              # within the original context: unchanged
    dyn_long = rope_cos_sin_table(D, 128, base, {"type": "dynamic", "factor": 2.0, "original_max_position_embeddings": 32})
    nb = base * ((2.0 * 128 / 32) - 1.0) ** (D / (D - 2))
    assert torch.allclose(dyn_long[7, 1], torch.tensor(math.cos(7 / nb ** (2 / D)), dtype=torch.float32), atol=1e-6)
    yarn = rope_cos_sin_table(D, N, base, {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 16, "mscale": 1.0,
                                           "mscale_all_dim": 0.0})
    assert float(yarn[0, 0]) == pytest.approx(0.1 * math.log(4.0) + 1.0, rel=1e-6)    # cos(0) times the attention factor


def test_shipped_model_extra_configs_load():
    """The sample ``MODEL_EXTRA_CFG_PATH`` files of the package load through the same reader as a user's and reach the
    engine configuration (reference: tests/test_config/*.json)."""
    import glob
    import os
    from omni_infer_b200 import config as oc
    from omni_infer_b200.adaptors.vllm.platform import ConfigUpdater
    from omni_infer_b200.engine.engine_core import EngineConfig
    root = os.path.join(os.path.dirname(oc.__file__), "configs")
    files = sorted(glob.glob(os.path.join(root, "*.json")))
    assert [os.path.basename(f) for f in files] == ["decode_ep8.json", "decode_ep8_placement.json", "prefill_ep8.json"]
    for f in files:
        extra = oc.load_model_extra_config(f)
        assert extra.parall_config.dp_size == 8
    dec = oc.load_model_extra_config(files[0])
    assert dec.operator_opt_config.moe_dispatch_combine and dec.operator_opt_config.decode_gear_list == [256]
    pre = oc.load_model_extra_config(files[2])
    assert pre.parall_config.dense_mlp_tp_size == 4 and not pre.operator_opt_config.moe_dispatch_combine
    pl = oc.load_model_extra_config(files[1])
    assert pl.operator_opt_config.use_omni_placement and pl.operator_opt_config.omni_placement_config_path.endswith("config.yaml")
