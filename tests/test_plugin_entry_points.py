"""The plugin surface: pyproject.toml declares the host engine's entry-point groups (``vllm.platform_plugins``,
``vllm.general_plugins``) and the ``omni_cli`` script (reference: pyproject.toml:17-27).  The tests install nothing:
they write the distribution's metadata directory from pyproject.toml into a temporary path entry, which is exactly
what the host engine's plugin loader (``importlib.metadata.entry_points(group=...)``) reads."""
import importlib
import importlib.metadata as md
import os
import sys
import tomllib

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture()
def dist_info(tmp_path, monkeypatch):
    proj = tomllib.load(open(os.path.join(ROOT, "pyproject.toml"), "rb"))["project"]
    d = tmp_path / f"{proj['name']}-{proj['version']}.dist-info"
    d.mkdir()
    (d / "METADATA").write_text(f"Metadata-Version: 2.1\nName: {proj['name']}\nVersion: {proj['version']}\n")
    lines = ["[console_scripts]"] + [f"{k} = {v}" for k, v in proj["scripts"].items()]
    for group, eps in proj["entry-points"].items():
        lines += ["", f"[{group}]"] + [f"{k} = {v}" for k, v in eps.items()]
    (d / "entry_points.txt").write_text("\n".join(lines) + "\n")
    monkeypatch.syspath_prepend(str(tmp_path))
    monkeypatch.setenv("NO_GPU_MOCK", "1")
    importlib.invalidate_caches()
    return proj


def test_platform_plugin_is_discovered_and_resolves(dist_info):
    eps = [e for e in md.entry_points(group="vllm.platform_plugins") if e.name == "b200"]
    assert len(eps) == 1
    qualname = eps[0].load()()
    assert qualname == "omni_infer_b200.adaptors.vllm.platform.B200Platform"
    mod, cls = qualname.rsplit(".", 1)
    platform = getattr(importlib.import_module(mod), cls)
    assert platform.get_worker_cls() == "omni_infer_b200.adaptors.vllm.worker.B200Worker"
    assert platform.get_attn_backend_cls(True).endswith("MLAAttention")
    try:
        from vllm.platforms.interface import Platform, PlatformEnum
    except Exception:  # noqa: BLE001
        pytest.skip("no host engine installed: the class stands alone")
    assert issubclass(platform, Platform) and platform._enum == PlatformEnum.OOT
    assert platform().is_out_of_tree()


def test_host_engine_loader_sees_the_plugins(dist_info):
    try:
        from vllm.plugins import load_plugins_by_group
    except Exception:  # noqa: BLE001
        pytest.skip("no host engine installed")
    found = load_plugins_by_group("vllm.platform_plugins")
    assert "b200" in found and found["b200"]() .endswith("B200Platform")
    general = load_plugins_by_group("vllm.general_plugins")
    assert {"b200_optimized_models", "kv_connectors"} <= set(general)
    models = general["b200_optimized_models"]()
    assert {"DeepseekV3ForCausalLM", "DeepseekV2ForCausalLM", "Qwen2ForCausalLM", "DeepSeekMTPModel"} <= set(models)
    from vllm import ModelRegistry
    import vllm.model_executor.models.registry as host_registry
    lazy = ModelRegistry.models["DeepseekV3ForCausalLM"]         # the host's entry now names this package's class
    assert getattr(lazy, "module_name", "").startswith("omni_infer_b200.models") and lazy.class_name == "DeepseekV3ForCausalLM"
    assert "Qwen3MoeForCausalLM" in ModelRegistry.get_supported_archs() and host_registry is not None
    conns = general["kv_connectors"]()
    assert "B200PeerPushConnectorV1" in conns and "AscendHcclConnectorV1" in conns
    from omni_infer_b200.accelerators.pd import get_connector_class
    assert get_connector_class("AscendHcclConnectorV1").__name__ == "WorkerConnector"


def test_check_and_update_config_on_a_host_engine_config(dist_info):
    from types import SimpleNamespace

    from omni_infer_b200.adaptors.vllm.platform import B200Platform
    vc = SimpleNamespace(parallel_config=SimpleNamespace(worker_cls="auto"), cache_config=SimpleNamespace(block_size=None),
                         scheduler_config=SimpleNamespace(scheduler_cls=None),
                         additional_config={"enable_hybrid_graph_mode": True})
    B200Platform.check_and_update_config(vc)
    assert vc.parallel_config.worker_cls.endswith("B200Worker") and vc.cache_config.block_size == 128
    assert vc.scheduler_config.scheduler_cls.endswith("engine.scheduler.Scheduler")


def test_cli_script_entry(dist_info):
    eps = {e.name: e for e in md.entry_points(group="console_scripts")}
    assert eps["omni_cli"].load().__module__ == "omni_infer_b200.cli.main"


def test_pangu_parsers_register_with_the_host_engine():
    """``register_model`` (the general-plugins hook) also puts the Pangu reasoning and tool-call parsers under the name
    ``pangu`` into the host engine's parser managers, and the adapters speak the managers' interface."""
    pytest.importorskip("vllm")
    from omni_infer_b200.models.pangu.host_engine import (PanguHostReasoningParser, PanguHostToolParser,
                                                          register_with_host_engine)
    done = register_with_host_engine()
    if done["reasoning"]:
        from vllm.reasoning import ReasoningParserManager
        assert ReasoningParserManager.get_reasoning_parser("pangu") is PanguHostReasoningParser
    if done["tool"]:
        from vllm.tool_parsers import ToolParserManager
        assert ToolParserManager.get_tool_parser("pangu") is PanguHostToolParser
    assert done["reasoning"] or done["tool"]

    class Tok:
        def get_vocab(self):
            return {"[unused16]": 7, "[unused17]": 8, "a": 1}

    r = PanguHostReasoningParser(Tok())
    assert r.extract_reasoning("[unused16]think[unused17]answer", None) == ("think", "answer")
    assert r.is_reasoning_end([1, 8, 1]) and not r.is_reasoning_end([1, 1]) and r.extract_content_ids([1, 8, 1, 1]) == [1, 1]
    d = r.extract_reasoning_streaming("[unused16]thi", "[unused16]think", "nk")
    assert (getattr(d, "reasoning", None) or (d.get("reasoning_content") if isinstance(d, dict) else None)) == "nk"
    t = PanguHostToolParser(Tok())
    ex = t.extract_tool_calls('ok [unused11]f|{"a": 1}[unused12]', None)
    assert ex.tools_called and ex.tool_calls[0].function.name == "f" if hasattr(ex.tool_calls[0], "function") else ex.tool_calls[0].name == "f"


def test_quantisation_name_registers_with_the_host_engine():
    pytest.importorskip("vllm")
    from omni_infer_b200.quantization.host_engine import NAME, register_with_host_engine
    if not register_with_host_engine():
        pytest.skip("the host engine's quantisation registry is not importable here")
    from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, get_quantization_config
    assert NAME in QUANTIZATION_METHODS
    cls = get_quantization_config(NAME)
    cfg = cls.from_config({"config_groups": {"group_0": {"weights": {"num_bits": 8}}}, "ignore": ["lm_head"]})
    assert cfg.get_name() == NAME and cfg.inner.name == "w8a8_int8" and cfg.inner.ignore == ["lm_head"]
    assert cls.get_config_filenames() == ["quant_model_description.json"] and cls.get_min_capability() == 100
    assert register_with_host_engine()                  # a second call is harmless


def test_connector_class_for_the_host_engine_delegates_to_the_pair():
    """The class the host engine's connector factory loads: one object per role over this package's connector pair; a
    prefill-role and a decode-role object move a request's blocks between two caches through the factory's interface."""
    pytest.importorskip("vllm")
    import time
    from types import SimpleNamespace
    import torch
    from vllm.distributed.kv_transfer.kv_connector.factory import KVConnectorFactory
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorBase_V1, KVConnectorRole
    from omni_infer_b200.accelerators import pd
    from omni_infer_b200.engine.request import Request, RequestStatus, SamplingParams
    pd.register()
    pd.InProcessHub.reset()
    loader = KVConnectorFactory._registry["B200PeerPushConnectorV1"]
    cls = loader()
    assert issubclass(cls, KVConnectorBase_V1) and cls.__name__ == "B200PeerPushConnectorV1"
    assert KVConnectorFactory._registry["AscendHcclConnectorV1"]() is cls

    def make(role_name, name):
        vc = SimpleNamespace(kv_transfer_config={"kv_role": role_name, "engine_id": name, "endpoint": f"inproc://{name}",
                                                 "sync_timeout_s": 5.0, "retries": 2, "retry_wait_s": 0.2},
                             cache_config=SimpleNamespace(block_size=4), speculative_config=None)
        return cls(vc, KVConnectorRole.WORKER, None)

    P, D = make("kv_producer", "hp"), make("kv_consumer", "hd")
    p_cache = {"layer0": torch.arange(8 * 4 * 2, dtype=torch.float32).view(8, 4, 2)}
    d_cache = {"layer0": torch.zeros(8, 4, 2)}
    P.register_kv_caches(p_cache)
    D.register_kv_caches(d_cache)
    # prefill side: a request that ended at its token cap hands blocks 2 and 3 over
    done = Request("r", list(range(7)), SamplingParams(max_tokens=1), status=RequestStatus.FINISHED_LENGTH_CAPPED, output_token_ids=[5])
    delay, params = P.request_finished(done, [2, 3])
    assert delay and params["remote_block_ids"] == [2, 3] and params["prefilled_token"] == 5
    # decode side: the scheduler reserves blocks 5 and 6 and asks for the load
    req = Request("r", list(range(7)), SamplingParams(max_tokens=4), kv_transfer_params=dict(params))
    n, is_async = D.get_num_new_matched_tokens(req, 0)
    assert (n, is_async) == (8, True)
    req.block_ids = [5, 6]
    D.update_state_after_alloc(req, SimpleNamespace(get_block_ids=lambda: [[5, 6]]), n)
    meta = D.build_connector_meta(None)
    D.bind_connector_metadata(meta)
    D.start_load_kv(None)
    sent = received = None
    for _ in range(200):
        s, r = D.get_finished(set())
        received = received or r
        s2, _ = P.get_finished(set())
        sent = sent or s2
        if sent and received:
            break
        time.sleep(0.01)
    assert received == {"r"} and sent == {"r"}
    assert torch.equal(d_cache["layer0"][5:7], p_cache["layer0"][2:4]) and float(d_cache["layer0"][:5].abs().sum()) == 0
    P.shutdown()
    D.shutdown()
    pd.InProcessHub.reset()
