"""Serving stack on CPU: API server (stream / non-stream, token counters, prefill hand-off fields), tokenizer pool,
deployment-file transform, launcher liveness handling, CLI dry run."""
import json
import sys
import time
import urllib.request

import pytest
import yaml

from omni_infer_b200.cli import main as cli_main
from omni_infer_b200.cli.config_transform import transform_deployment_config
from omni_infer_b200.cli.launch import Launcher, dp_rank_env
from omni_infer_b200.engine.api_server import serve
from omni_infer_b200.engine.engine_core import EngineConfig
from omni_infer_b200.engine.tokenizer_pool import TokenizerPool


def _post(port, path, body, stream=False):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=30) as r:
        return r.read().decode()


def test_api_server_completions_and_stream():
    from omni_infer_b200.accelerators.pd import InProcessHub
    InProcessHub.reset()
    cfg = EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu",
                       kv_transfer_config={"kv_role": "kv_producer", "engine_id": "api-p", "endpoint": "inproc://api-p"})
    srv, aeng = serve(cfg, "127.0.0.1", 0, block=False)
    port = srv.server_port
    try:
        r = json.loads(_post(port, "/v1/completions", {"prompt": "hello world", "max_tokens": 5}))
        assert r["usage"]["completion_tokens"] == 5 and r["prompt_num_token"] == 11 and r["output_num_token"] == 5
        text = _post(port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True})
        chunks = [json.loads(l[6:]) for l in text.splitlines() if l.startswith("data: {")]
        assert chunks[-1]["output_num_token"] == 4 and chunks[-1]["usage"]["total_tokens"] == chunks[-1]["prompt_num_token"] + 4
        assert "[DONE]" in text and chunks[-1]["choices"][0]["finish_reason"] == "length"
        # a client that asks for it gets a closing chunk without choices that carries the request's totals
        text = _post(port, "/v1/completions", {"prompt": "hi", "max_tokens": 3, "stream": True, "stream_options": {"include_usage": True}})
        chunks = [json.loads(l[6:]) for l in text.splitlines() if l.startswith("data: {")]
        assert chunks[-1]["choices"] == [] and chunks[-1]["usage"] == {"prompt_tokens": 2, "completion_tokens": 3, "total_tokens": 5}
        assert chunks[-2]["choices"][0]["finish_reason"] == "length" and text.rstrip().endswith("[DONE]")
        # prefill leg of a PD request: one token, hand-off parameters in the response
        r = json.loads(_post(port, "/v1/completions", {"prompt": [1, 2, 3, 4, 5], "max_tokens": 1,
                                                       "kv_transfer_params": {"do_remote_decode": True}}))
        kv = r["kv_transfer_params"]
        assert kv["prompt_token_ids"] == [1, 2, 3, 4, 5] and kv["remote_block_ids"] and kv["prefilled_token"] is not None
        m = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
        assert "omni_requests_total 4" in m
    finally:
        srv.shutdown()
        aeng.stop()
        InProcessHub.reset()


def _status(port, path, body):
    import urllib.error
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=30) as r:
            return r.status, json.loads(r.read().decode())
    except urllib.error.HTTPError as e:
        return e.code, json.loads(e.read().decode() or "{}")


def _status_id(port, body, rid):
    import urllib.error
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json", "X-Request-Id": rid})
    try:
        with urllib.request.urlopen(req, timeout=30) as r:
            return r.status, json.loads(r.read().decode())
    except urllib.error.HTTPError as e:
        return e.code, json.loads(e.read().decode() or "{}")


def test_api_server_refuses_bad_input_drops_disconnected_clients_and_reports_a_failing_engine():
    import socket
    import urllib.error
    cfg = EngineConfig(block_size=16, num_kv_blocks=8, max_model_len=64, device="cpu")
    srv, aeng = serve(cfg, "127.0.0.1", 0, block=False)
    port = srv.server_port
    eng = aeng.engine
    try:
        # ---- input that cannot be served is answered at once, not after a time-out
        assert _status(port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": "many"})[0] == 400
        assert _status(port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": 4, "top_p": 1.5})[0] == 400
        assert _status(port, "/v1/completions", {"prompt": [], "max_tokens": 4})[0] == 400
        for bad in (0, -3, 2.5, True):                     # zero is not "use the default"
            assert _status(port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": bad})[0] == 400, bad
        code, err = _status(port, "/v1/completions", {"prompt": list(range(70)), "max_tokens": 4})
        assert code == 400 and "context" in err["error"]
        # ---- a body that is not an object, or whose length is not a number, is refused without a stack trace
        assert _status(port, "/v1/completions", [1, 2, 3])[0] == 400
        bad_len = socket.create_connection(("127.0.0.1", port))
        bad_len.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Length: many\r\n\r\n{}")
        assert bad_len.recv(200).split(b"\r\n")[0].endswith(b"400 Bad Request")
        bad_len.close()
        # ---- shapes the server does not serve are refused, not guessed at; token ids outside the table never reach the model
        for body in ({"prompt": ["a", "b"]}, {"prompt": None}, {"prompt": [[1, 2], [3]]}, {"prompt": [1, 2], "n": 2},
                     {"prompt": [1, 2], "logprobs": 5}, {"prompt": [1, -5]}, {"prompt": [1, 10 ** 9]},
                     {"prompt": [1, 2], "kv_transfer_params": "x"}, {"prompt": "x", "kv_transfer_params": {"prompt_token_ids": [1, 10 ** 9]}}):
            assert _status(port, "/v1/completions", body)[0] == 400, body
        for body in ({"messages": "hi"}, {"messages": [1, 2]}):
            assert _status(port, "/v1/chat/completions", body)[0] == 400, body
        assert _status(port, "/v1/completions", {"prompt": ["one prompt"], "max_tokens": 1})[0] == 200      # a batch of one
        parts = {"messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}], "max_tokens": 1}
        plain = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 1}
        a, b = _status(port, "/v1/chat/completions", parts), _status(port, "/v1/chat/completions", plain)
        assert a[0] == b[0] == 200 and a[1]["usage"]["prompt_tokens"] == b[1]["usage"]["prompt_tokens"]
        with pytest.raises(ValueError):
            eng.add_request([1, 5000])
        # ---- a fault inside the handler itself is answered (500), and the server goes on serving
        real_submit = aeng.submit

        def boom(*a, **k):
            raise KeyError("boom")
        aeng.submit = boom
        code, err = _status(port, "/v1/completions", {"prompt": [1, 2], "max_tokens": 2})
        assert code == 500 and "KeyError" in err["error"]
        aeng.submit = real_submit
        assert _status(port, "/v1/completions", {"prompt": [1, 2], "max_tokens": 2})[0] == 200
        # ---- the small endpoints clients and load generators ask first
        models = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/models", timeout=5).read())
        assert models["data"][0]["id"] and models["data"][0]["max_model_len"] == 64
        import omni_infer_b200
        assert json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/version", timeout=5).read())["version"] == omni_infer_b200.__version__
        code, t = _status(port, "/tokenize", {"prompt": "héllo"})
        assert code == 200 and t["count"] == len(t["tokens"]) == 6
        assert _status(port, "/detokenize", {"tokens": t["tokens"]}) == (200, {"prompt": "héllo"})
        assert _status(port, "/detokenize", {"tokens": "abc"})[0] == 400 and _status(port, "/tokenize", {"prompt": 5})[0] == 400
        metrics = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
        assert "omni_engine_healthy 1" in metrics and "omni_failed_steps_total 0" in metrics
        # a prompt that fits the context but not the KV pool (7 usable blocks of 16 tokens) is ended by the scheduler,
        # and the client hears about it
        big = EngineConfig(block_size=16, num_kv_blocks=4, max_model_len=128, device="cpu")
        srv2, aeng2 = serve(big, "127.0.0.1", 0, block=False)
        try:
            t0 = time.time()
            code, err = _status(srv2.server_port, "/v1/completions", {"prompt": list(range(100)), "max_tokens": 4})
            assert code == 500 and "does not fit" in err["error"] and time.time() - t0 < 10
            assert _status(srv2.server_port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": 2})[0] == 200
        finally:
            srv2.shutdown()
            aeng2.stop()
        # ---- a client that goes away while its (non-streaming) request runs: the request is dropped from the engine
        real_step = eng.step
        eng.step = lambda: (time.sleep(0.05), real_step())[1]          # slow the engine down a little
        s = socket.create_connection(("127.0.0.1", port))
        body = json.dumps({"prompt": [5, 6, 7], "max_tokens": 60, "ignore_eos": True}).encode()
        s.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: "
                  + str(len(body)).encode() + b"\r\n\r\n" + body)
        for _ in range(100):
            if eng.scheduler.num_running:
                break
            time.sleep(0.02)
        assert eng.scheduler.num_running == 1
        s.close()
        for _ in range(200):
            if not eng.has_unfinished:
                break
            time.sleep(0.02)
        req = list(eng.scheduler.requests.values())[-1]              # the one whose client went away
        assert not eng.has_unfinished and req.status.name == "FINISHED_ABORTED" and len(req.output_token_ids) < 60
        assert not aeng.queues                              # the output queue of the dropped request went with it
        # ---- a request id that is still in flight is refused; once that request has ended the id can be used again
        import threading
        first = {}
        t = threading.Thread(target=lambda: first.update(r=_status_id(port, {"prompt": [5, 6], "max_tokens": 30, "ignore_eos": True}, "same")))
        t.start()
        for _ in range(100):
            if "same" in aeng.queues:
                break
            time.sleep(0.02)
        assert _status_id(port, {"prompt": [5, 6], "max_tokens": 2}, "same")[0] == 409
        t.join()
        assert first["r"][0] == 200 and first["r"][1]["usage"]["completion_tokens"] == 30
        assert _status_id(port, {"prompt": [5, 6], "max_tokens": 2}, "same")[0] == 200
        eng.step = real_step
        # ---- an engine whose steps fail: requests get an error, are dropped, and /health turns 503 until a step works
        assert urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5).status == 200

        def broken():
            raise RuntimeError("device lost")
        eng.step = broken
        for _ in range(aeng.UNHEALTHY_AFTER):
            code, err = _status(port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": 4})
            assert code == 500 and "engine failure" in err["error"]
        assert not eng.scheduler.running and not eng.scheduler.waiting          # nothing left to fail again
        with pytest.raises(urllib.error.HTTPError) as ei:
            urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5)
        assert ei.value.code == 503
        eng.step = real_step
        assert _status(port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": 2})[0] == 200
        assert urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5).status == 200
    finally:
        srv.shutdown()
        aeng.stop()


def test_api_sampling_parameters_and_stop_strings():
    """Penalties, seeds and stop token ids reach the sampler, and stop strings end a request at the text level: the
    answer stops before the string, in both response forms."""
    cfg = EngineConfig(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu")
    srv, aeng = serve(cfg, "127.0.0.1", 0, block=False)
    port = srv.server_port
    try:
        plain = json.loads(_post(port, "/v1/completions", {"prompt": "hello world", "max_tokens": 12}))
        text = plain["choices"][0]["text"]
        assert plain["usage"]["completion_tokens"] == 12 and len(text) >= 6
        # a strong repetition penalty changes the greedy continuation
        pen = json.loads(_post(port, "/v1/completions", {"prompt": "hello world", "max_tokens": 12, "repetition_penalty": 50.0}))
        assert pen["choices"][0]["text"] != text
        # stop token id = the third generated token of the plain run: two tokens come back
        from omni_infer_b200.engine.tokenizer_pool import ByteTokenizer
        ids = ByteTokenizer(1024).encode(text)
        # (the byte tokenizer maps characters to ids one to one for ASCII; otherwise take the ids from the engine)
        req = next(r for r in aeng.engine.scheduler.requests.values() if len(r.output_token_ids) == 12 and r.sampling.repetition_penalty == 1.0)
        third = req.output_token_ids[2]
        short = json.loads(_post(port, "/v1/completions", {"prompt": "hello world", "max_tokens": 12, "stop_token_ids": [third]}))
        assert short["usage"]["completion_tokens"] <= 3 and short["choices"][0]["finish_reason"] == "stop"
        # stop string taken from the middle of the plain answer
        needle = text[4:6]
        cut = json.loads(_post(port, "/v1/completions", {"prompt": "hello world", "max_tokens": 12, "stop": needle}))
        assert cut["choices"][0]["text"] == text[:text.find(needle)] and cut["choices"][0]["finish_reason"] == "stop"
        streamed = _post(port, "/v1/completions", {"prompt": "hello world", "max_tokens": 12, "stop": [needle], "stream": True})
        chunks = [json.loads(l[6:]) for l in streamed.splitlines() if l.startswith("data: {")]
        assert "".join(c["choices"][0]["text"] for c in chunks) == text[:text.find(needle)]
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and "[DONE]" in streamed
        for _ in range(100):
            if not aeng.engine.has_unfinished:
                break
            time.sleep(0.02)
        assert not aeng.engine.has_unfinished            # the stopped requests left the engine
        assert _status(port, "/v1/completions", {"prompt": "x", "max_tokens": 2, "repetition_penalty": -1})[0] == 400
        assert _status(port, "/v1/completions", {"prompt": "x", "max_tokens": 2, "priority": "soon"})[0] == 400
    finally:
        srv.shutdown()
        aeng.stop()


def test_chat_endpoint_splits_reasoning_content_and_tool_calls():
    """The chat endpoint with ``--reasoning-parser pangu --tool-call-parser pangu``: a scripted model answer with a
    chain of thought, an answer and a tool call comes back as reasoning_content / content / tool_calls, whole and
    streamed (the markers never reach the client, also when they arrive split over several tokens)."""
    import queue
    import threading
    from http.server import ThreadingHTTPServer
    from types import SimpleNamespace
    from omni_infer_b200.engine.api_server import _make_parsers, make_handler
    from omni_infer_b200.engine.request import RequestOutput
    script = '[unused16]the user wants weather[unused17]Let me check. [unused11]get_weather|{"city": "Paris"}[unused12]'
    data = list(script.encode())

    class FakeEngine:
        stats = {"requests": 0, "tokens": 0, "failed_steps": 0}
        healthy = True
        engine = SimpleNamespace(role="mixed", cfg=SimpleNamespace(max_model_len=4096))

        def submit(self, ids, sp, rid, kvp=None, priority=0):
            q = queue.Queue()
            for i in range(0, len(data), 3):               # three bytes per step: markers are split across steps
                chunk = data[i:i + 3]
                last = i + 3 >= len(data)
                q.put(RequestOutput(rid, chunk, last, "stop" if last else None, None, len(ids), i + len(chunk)))
            return q

        def abort(self, rid):
            pass

    with pytest.raises(ValueError):
        _make_parsers("nope", None)
    reasoning, tools = _make_parsers("pangu", "pangu")
    tok = TokenizerPool(None, vocab_size=1024)
    srv = ThreadingHTTPServer(("127.0.0.1", 0), make_handler(FakeEngine(), tok, "m", reasoning, tools))
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    port = srv.server_port
    try:
        body = {"messages": [{"role": "user", "content": "weather in Paris?"}], "max_tokens": 200}
        r = json.loads(_post(port, "/v1/chat/completions", body))
        msg = r["choices"][0]["message"]
        assert msg["reasoning_content"] == "the user wants weather" and msg["content"] == "Let me check."
        assert msg["tool_calls"][0]["function"] == {"name": "get_weather", "arguments": '{"city": "Paris"}'}
        assert r["choices"][0]["finish_reason"] == "tool_calls"
        text = _post(port, "/v1/chat/completions", dict(body, stream=True))
        chunks = [json.loads(l[6:]) for l in text.splitlines() if l.startswith("data: {")]
        deltas = [c["choices"][0]["delta"] for c in chunks]
        assert "".join(d.get("reasoning_content", "") for d in deltas) == "the user wants weather"
        assert "".join(d.get("content", "") for d in deltas).strip() == "Let me check."
        calls = [t for d in deltas for t in d.get("tool_calls", [])]
        assert len(calls) == 1 and calls[0]["function"]["name"] == "get_weather" and calls[0]["index"] == 0
        assert "unused" not in "".join(json.dumps(d) for d in deltas)
        assert chunks[-1]["choices"][0]["finish_reason"] == "tool_calls"
        # the plain completions endpoint is not touched by the parsers
        r = json.loads(_post(port, "/v1/completions", {"prompt": "x", "max_tokens": 200}))
        assert r["choices"][0]["text"] == script
    finally:
        srv.shutdown()
        tok.shutdown()


def test_tokenizer_pool_offloads_long_prompts():
    pool = TokenizerPool(None, vocab_size=300, workers=1, threshold=10, enabled=True)
    try:
        assert pool.encode("short") == [ord(c) for c in "short"]
        long = "x" * 50
        assert pool.encode(long) == [ord("x")] * 50
        assert TokenizerPool._parse_cores("0-2,5") == {0, 1, 2, 5}
    finally:
        pool.shutdown()


DEPLOY = {
    "deployment": {
        "prefill": {"group1": [{"ip": "127.0.0.1", "devices": "0,1", "api_port": 9000}, {"ip": "127.0.0.1", "devices": "2,3", "api_port": 9001}]},
        "decode": {"group1": [{"ip": "127.0.0.1", "ascend_rt_visible_devices": "4,5,6,7", "api_port": 9100}]},
        "proxy": {"ip": "127.0.0.1", "listen_port": 8080, "prefill_lb_sdk": "prefill_score_balance", "decode_lb_sdk": "weighted_least_active"},
    },
    "services": {"model_path": "deepseek-v3", "prefill": {"max_model_len": 32000}, "decode": {"max_model_len": 16384, "num_speculative_tokens": 1,
                 "additional_config": {"multi_step": 2}}},
}


def test_tokenizer_pool_survives_a_dead_worker():
    import os
    import signal
    pool = TokenizerPool(None, vocab_size=1024, workers=1, threshold=8, enabled=True)
    try:
        text = "a fairly long prompt " * 4
        want = pool.tokenizer.encode(text)
        assert pool.encode(text) == want
        (pid,) = list(pool.pool._processes)                  # the one worker
        os.kill(pid, signal.SIGKILL)
        time.sleep(0.2)
        assert pool.encode(text) == want                     # tokenised here, pool replaced
        assert pool.pool_restarts == 1
        assert pool.encode(text) == want and pool.pool_restarts == 1      # and the new pool works
    finally:
        pool.shutdown()


def test_deployment_transform_and_cli_dry_run(tmp_path, capsys):
    procs = transform_deployment_config(DEPLOY)
    assert [p.role for p in procs] == ["prefill", "prefill", "decode", "proxy"]
    assert procs[0].env["CUDA_VISIBLE_DEVICES"] == "0,1" and procs[2].env["CUDA_VISIBLE_DEVICES"] == "4,5,6,7"
    assert "--enforce-eager" in procs[0].argv and "--num-speculative-tokens" in procs[2].argv
    px = procs[3].argv
    assert px[px.index("--prefill-servers-list") + 1] == "127.0.0.1:9000,127.0.0.1:9001"
    assert px[px.index("--decode-lb-sdk") + 1] == "weighted_least_active"
    kv = json.loads(procs[2].argv[procs[2].argv.index("--kv-transfer-config") + 1])
    assert kv["kv_role"] == "kv_consumer" and kv["transport"] == "tcp"
    f = tmp_path / "deploy.yml"
    f.write_text(yaml.safe_dump(DEPLOY))
    assert cli_main.main(["serve", str(f), "--dry-run"]) == 0
    assert len(json.loads(capsys.readouterr().out)) == 4
    assert cli_main.main(["status", "--config", str(f)]) == 1          # nothing is listening
    env = dp_rank_env(3, 8)
    assert env["VLLM_DP_RANK"] == "3" and env["WORLD_SIZE"] == "8"


def test_inventory_and_playbook_for_several_hosts(tmp_path, capsys):
    """The deployment file as an ansible inventory (host groups P / D / C with the process each host runs) and the
    playbook that uses it: every variable a task reads is an inventory variable or has a default, the tags are the
    reference's, and the topology step calls the topology tool with options it has."""
    import os
    import re
    from omni_infer_b200.accelerators.pd import topology
    from omni_infer_b200.cli.config_transform import plan_to_inventory
    dep = json.loads(json.dumps(DEPLOY))
    dep["deployment"]["prefill"]["group1"][0]["ip"] = "10.0.0.1"
    dep["deployment"]["decode"]["group1"][0]["ip"] = "10.0.0.3"
    inv = plan_to_inventory(dep)
    groups = inv["all"]["children"]
    assert list(groups) == ["P", "D", "C"]
    p0, d0, c0 = groups["P"]["hosts"]["p0"], groups["D"]["hosts"]["d0"], groups["C"]["hosts"]["c0"]
    assert p0["ansible_host"] == "10.0.0.1" and p0["devices"] == "0,1" and p0["kv_rank"] == 0 and p0["node_rank"] == 0
    assert groups["P"]["hosts"]["p1"]["kv_rank"] == 1 and groups["P"]["hosts"]["p1"]["node_rank"] == 1
    assert d0["ansible_host"] == "10.0.0.3" and d0["server_env"]["ROLE"] == "decode" and "--num-speculative-tokens" in d0["server_argv"]
    assert "10.0.0.1:9000" in " ".join(c0["proxy_argv"]) and c0["listen_port"] == 8080
    f = tmp_path / "deploy.yml"
    f.write_text(yaml.safe_dump(dep))
    out = tmp_path / "inv.yml"
    assert cli_main.main(["inventory", str(f), "-o", str(out)]) == 0
    assert yaml.safe_load(out.read_text()) == inv
    capsys.readouterr()
    cwd = os.getcwd()
    os.chdir(tmp_path)
    try:
        assert cli_main.main(["serve", str(f), "--ansible", "--dry-run"]) == 0
    finally:
        os.chdir(cwd)
    plan = json.loads(capsys.readouterr().out)
    assert plan["command"][0] == "ansible-playbook" and plan["command"][-1].endswith("omni_infer_server.yml")
    # ---- the playbook
    path = os.path.join(os.path.dirname(cli_main.__file__), "omni_infer_server.yml")
    text = open(path).read()
    plays = yaml.safe_load(text)
    tags = {t for play in plays for t in play["tags"]}
    assert {"run_docker", "sync_code", "topology", "run_server", "run_proxy", "fetch_log", "stop"} <= tags
    assert all(play["hosts"] in ("P:D:C", "P:D", "C") for play in plays)
    known = set(inv["all"]["vars"]) | set(p0) | set(c0) | {"inventory_hostname", "playbook_dir", "health", "k", "v"}
    used = set()
    for expr in re.findall(r"{{(.*?)}}|{%(.*?)%}", text):
        body = expr[0] or expr[1]
        if "default(" in body:
            continue
        body = re.sub(r"'[^']*'", "", body)                       # string literals
        used |= {w for w in re.findall(r"[A-Za-z_][A-Za-z_0-9]*", body)
                 if w not in ("if", "else", "for", "in", "endfor", "map", "join", "quote", "items", "status")}
    assert used <= known, used - known
    # the topology step's options exist in the tool, and a table per host merges into one
    opts = set(re.findall(r"(--[a-z-]+)", text[text.index("tags: [topology]"):text.index("tags: [run_server]")]))
    assert opts <= {"--mode", "--prefill-server-list", "--decode-server-list", "--host", "--base-api-port", "--base-control-port",
                    "--save-dir", "--global-ranktable-list", "--index-offset"}
    for name, h in list(groups["P"]["hosts"].items()) + list(groups["D"]["hosts"].items()):
        role_opt = "--prefill-server-list" if h["role"] == "prefill" else "--decode-server-list"
        off = 0 if h["role"] == "prefill" else 100
        assert topology.main(["--mode", "gen", role_opt, h["devices"], "--host", h["ansible_host"], "--index-offset",
                              str(h["kv_rank"]), "--base-api-port",
                              str(h["api_port"] - off), "--base-control-port", str(h["control_port"] - off),
                              "--save-dir", str(tmp_path / name)]) == 0
    tables = [str(tmp_path / n / "global_topology.json") for n in ("p0", "p1", "d0")]
    assert topology.main(["--mode", "merge-all", "--global-ranktable-list", *tables, "--save-dir", str(tmp_path / "all")]) == 0
    merged = topology.Topology.load(str(tmp_path / "all" / "global_topology.json"))
    assert sorted((i.name, i.host, i.api_port) for i in merged.instances) == [
        ("decode-0", "10.0.0.3", 9100), ("prefill-0", "10.0.0.1", 9000), ("prefill-1", "127.0.0.1", 9001)]
    # the table's control endpoints are the ones the servers listen on (the connectors only talk to listed instances)
    listening = set()
    for h in list(groups["P"]["hosts"].values()) + list(groups["D"]["hosts"].values()):
        listening.add(json.loads(h["server_argv"][h["server_argv"].index("--kv-transfer-config") + 1])["endpoint"])
    assert merged.control_endpoints() == listening and len(listening) == 3
    # container image and build script exist and say what they build for
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    assert "deploy/build.sh" in open(os.path.join(root, "deploy", "docker", "Dockerfile")).read()
    assert "g.build()" in open(os.path.join(root, "deploy", "build.sh")).read()


def test_shipped_deployment_file_describes_a_runnable_plan(capsys):
    import os
    path = os.path.join(os.path.dirname(cli_main.__file__), "omni_infer_deployment.yml")
    procs = transform_deployment_config(path)
    assert [p.role for p in procs] == ["prefill"] * 4 + ["decode"] * 4 + ["proxy"]
    assert sorted(p.env["CUDA_VISIBLE_DEVICES"] for p in procs[:8]) == [str(i) for i in range(8)]     # every GPU once
    assert len({p.api_port for p in procs}) == 9
    ends = [json.loads(p.argv[p.argv.index("--kv-transfer-config") + 1])["endpoint"] for p in procs[:8]]
    assert len(set(ends)) == 8
    assert cli_main.main(["serve", path, "--dry-run"]) == 0
    assert len(json.loads(capsys.readouterr().out)) == 9


def test_launcher_detects_dead_child(tmp_path):
    from omni_infer_b200.cli.config_transform import ProcessSpec
    procs = [ProcessSpec("sleeper", "decode", ["-c", "import time; time.sleep(30)"]),
             ProcessSpec("crasher", "prefill", ["-c", "import sys; sys.exit(3)"])]
    la = Launcher(procs, str(tmp_path))
    la.start()
    try:
        dead = []
        for _ in range(100):
            dead += la.poll()
            if dead:
                break
            time.sleep(0.05)
        assert dead == ["crasher"] and "sleeper" in la.children
    finally:
        la.stop()
    assert not la.children


def test_pd_run_and_qwen_one_click_plans(tmp_path):
    """The launchers keep the reference's option names: per-DP-rank servers with the DP environment, KV roles by
    instance role, hardware-specific options accepted and ignored, and the one-click Qwen layouts."""
    import json as _json

    from omni_infer_b200.cli import pd_run, run_model_qwen
    a = pd_run.parse(["--role", "decode", "--num-servers", "2", "--num-dp", "4", "--server-offset", "2", "--base-api-port", "19001",
                      "--master-ip", "127.0.0.1", "--master-port", "8503", "--rank-table-path", "x.json", "--hccl-buffsize", "200",
                      "--enable-mtp", "--num-speculative-tokens", "1", "--cuda-visible-devices", "4,5", "--extra-args=--enforce-eager"])
    plan = pd_run.build_plan(a)
    assert [p.env["VLLM_DP_RANK"] for p in plan] == ["2", "3"] and plan[0].env["VLLM_DP_SIZE"] == "4"
    assert plan[0].env["CUDA_VISIBLE_DEVICES"] == "4" and plan[1].env["CUDA_VISIBLE_DEVICES"] == "5"
    kv = _json.loads(plan[1].argv[plan[1].argv.index("--kv-transfer-config") + 1])
    assert kv["kv_role"] == "kv_consumer" and kv["engine_id"].endswith("-3")
    assert "--num-speculative-tokens" in plan[0].argv and plan[0].argv[-1] == "--enforce-eager"
    q = run_model_qwen.build_plan(run_model_qwen.parse(["--model-path", "qwen3-30b-a3b", "--deploy-mode", "pd_separate",
                                                        "--server-list", "0,1,2,3", "--service-port", "6660,6760"]))
    assert [p.role for p in q] == ["prefill", "prefill", "decode", "decode", "proxy"]
    assert "--prefill-servers-list" in q[-1].argv and q[2].api_port == 6760
    m = run_model_qwen.build_plan(run_model_qwen.parse(["--model-path", "qwen2-small", "--server-list", "0,1", "--graph-true", "true"]))
    assert [p.role for p in m] == ["mixed", "mixed", "proxy"] and "--enforce-eager" not in m[0].argv


def test_proxy_launcher_rolls_back_to_the_configuration_that_started(tmp_path):
    import json as _json
    import subprocess as sp
    import sys as _sys
    import time as _time

    base = [_sys.executable, "-m", "omni_infer_b200.accelerators.sched.global_proxy", "--pid-file", str(tmp_path / "pid"),
            "--state-dir", str(tmp_path / "state"), "--listen-host", "127.0.0.1", "--log-file", str(tmp_path / "proxy.log")]
    good = base + ["--listen-port", "18471", "--decode-servers-list", "127.0.0.1:18999"]
    dry = sp.run(good + ["--dry-run"], capture_output=True, text=True)
    info = _json.loads(dry.stdout)
    assert info["nofile"] == 65535 and any("somaxconn" in c for c in info["os_tuning"])
    try:
        assert sp.run(good, capture_output=True, text=True).returncode == 0
        st = _json.loads(sp.run(base + ["--decode-servers-list", "x:1", "--status"], capture_output=True, text=True).stdout)
        assert st["running"]
        sp.run(base + ["--decode-servers-list", "x:1", "--stop"], capture_output=True)
        _time.sleep(0.2)
        # a configuration that cannot start (port 1 needs privileges / is invalid): the launcher restarts the good one
        bad = base + ["--listen-port", "1", "--decode-servers-list", "127.0.0.1:18999"]
        r = sp.run(bad, capture_output=True, text=True)
        if r.returncode != 0:
            assert "rolled back" in r.stderr
            st = _json.loads(sp.run(base + ["--decode-servers-list", "x:1", "--status"], capture_output=True, text=True).stdout)
            assert st["running"] and "18471" in " ".join(st["config"]["command"])
    finally:
        sp.run(base + ["--decode-servers-list", "x:1", "--stop"], capture_output=True)


def test_request_timeline_joins_proxy_prefill_and_decode(tmp_path):
    """One request through the C++ proxy, a prefill engine and a decode engine: the three logs join on the request id
    into one ordered timeline, and the tool reports the stage intervals."""
    import subprocess
    from omni_infer_b200.accelerators.pd import InProcessHub
    from omni_infer_b200.build import PROXY_BIN, build_proxy
    from omni_infer_b200.utils import timeline

    InProcessHub.reset()
    eng_log, proxy_log = tmp_path / "engines.log", tmp_path / "proxy.log"
    assert timeline.configure(str(eng_log))
    build_proxy()
    kv = lambda role, name: {"kv_role": role, "engine_id": name, "endpoint": f"inproc://{name}"}
    base = dict(block_size=16, num_kv_blocks=32, max_model_len=128, device="cpu")
    p_srv, p_eng = serve(EngineConfig(kv_transfer_config=kv("kv_producer", "tl-p"), **base), "127.0.0.1", 0, block=False)
    d_srv, d_eng = serve(EngineConfig(kv_transfer_config=kv("kv_consumer", "tl-d"), **base), "127.0.0.1", 0, block=False)
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    with open(proxy_log, "w") as plog:
        proxy = subprocess.Popen([str(PROXY_BIN), "--listen", f"127.0.0.1:{port}", "--prefill-servers", f"127.0.0.1:{p_srv.server_port}",
                                  "--decode-servers", f"127.0.0.1:{d_srv.server_port}", "--log-level", "0", "--timeline"], stderr=plog)
        try:
            for _ in range(100):
                try:
                    urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=0.5).read()
                    break
                except Exception:
                    time.sleep(0.05)
            req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions",
                                         data=json.dumps({"prompt": list(range(1, 40)), "max_tokens": 4}).encode(),
                                         headers={"Content-Type": "application/json", "X-Request-Id": "tl-req-1"})
            out = json.loads(urllib.request.urlopen(req, timeout=60).read())
            assert out["usage"]["completion_tokens"] == 4
        finally:
            proxy.terminate()
            proxy.wait(timeout=10)
            for srv, eng in ((p_srv, p_eng), (d_srv, d_eng)):
                srv.shutdown()
                eng.stop()
            timeline.configure("")
            InProcessHub.reset()
    tl = timeline.parse([str(proxy_log), str(eng_log)])
    ev = tl["tl-req-1"]
    roles = [r for _, r, _ in ev]
    actions = [a for _, _, a in ev]
    assert {"proxy", "prefill", "decode"} <= set(roles)
    assert actions[0] == "Proxy got request" and actions[-1] == "Proxy finished request"
    pairs = list(zip(roles, actions))
    order = [("proxy", "Proxy sends to prefill"), ("prefill", "Get request in api server"), ("prefill", "Prefill scheduled"),
             ("prefill", "First token sampled"), ("proxy", "Proxy got prefill response"), ("proxy", "Proxy sends to decode"),
             ("decode", "Get request in api server"), ("decode", "First token out of api server"),
             ("decode", "Finish response in api server"), ("proxy", "Proxy relays first decode bytes")]   # not streamed
    pos = [pairs.index(x) for x in order]
    assert pos == sorted(pos), pairs
    assert any(r == "decode" and "pull kv" in a for r, a in pairs), pairs
    s = timeline.summary(tl)
    assert s["requests"] == 1 and s["end_to_end_ms"]["p50"] > 0
    assert "proxy:Proxy sends to prefill -> prefill:Get request in api server" in s["stages"]
    text = timeline.render(tl)
    assert "request tl-req-1" in text and "p50" in text
    assert timeline.main([str(proxy_log), str(eng_log), "--json", str(tmp_path / "s.json")]) == 0
    assert json.load(open(tmp_path / "s.json"))["requests"] == 1


def test_an_idle_prefill_server_releases_handed_over_blocks_without_new_traffic():
    """A prefill instance keeps a finished prompt's blocks for the decode side.  When the decode side never comes (its
    client hung up) they are released when the hand-over's time is up - also on a server that receives nothing else:
    its loop keeps stepping while hand-overs are outstanding."""
    from omni_infer_b200.accelerators.pd import InProcessHub
    InProcessHub.reset()
    cfg = EngineConfig(block_size=16, num_kv_blocks=8, max_model_len=64, device="cpu",
                       kv_transfer_config={"kv_role": "kv_producer", "engine_id": "idle-p", "endpoint": "inproc://idle-p",
                                           "handover_ttl_s": 0.5})
    srv, aeng = serve(cfg, "127.0.0.1", 0, block=False)
    eng = aeng.engine
    try:
        code, out = _status(srv.server_port, "/v1/completions", {"prompt": list(range(1, 30)), "max_tokens": 1})
        assert code == 200 and out["kv_transfer_params"]["remote_block_ids"]
        assert eng.scheduler.pending_free and eng.kv.num_free_blocks < eng.kv.num_blocks - 1
        for _ in range(100):
            if not eng.scheduler.pending_free:
                break
            time.sleep(0.05)
        assert not eng.scheduler.pending_free and eng.kv.num_free_blocks == eng.kv.num_blocks - 1
    finally:
        srv.shutdown()
        aeng.stop()
        InProcessHub.reset()
