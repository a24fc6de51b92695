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
