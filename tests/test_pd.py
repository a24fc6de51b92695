"""PD disaggregation on CPU: a prefill engine and a decode engine in one process, KV blocks pushed between their
paged caches, prefilled-token reuse, acknowledgement-driven block release, and host-side fault injection (dropped
and duplicated control messages, a transfer that never completes -> local-prefill fallback)."""
import time

import pytest
import torch

from omni_infer_b200.accelerators.pd import InProcessHub
from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
from omni_infer_b200.engine.request import SamplingParams


def _engine(role, name, **kw):
    cfg = EngineConfig(block_size=16, num_kv_blocks=kw.pop("num_kv_blocks", 48), max_model_len=160, device="cpu", seed=0,
                       kv_transfer_config={"kv_role": role, "engine_id": name, "endpoint": f"inproc://{name}",
                                           "sync_timeout_s": kw.pop("sync_timeout_s", 5.0), "retries": kw.pop("retries", 3),
                                           "retry_wait_s": kw.pop("retry_wait_s", 0.2)}, **kw)
    return EngineCore(cfg)


def _prompts(n=3, length=40, seed=4):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def _run_pd(P, D, prompts, max_tokens, deadline_s=30.0):
    # prefill instance: one token, KV kept
    for i, p in enumerate(prompts):
        P.add_request(p, SamplingParams(max_tokens=1), request_id=f"r{i}", kv_transfer_params={"do_remote_decode": True})
    handoff = {}
    while P.scheduler.has_unfinished:
        for out in P.step():
            if out.finished:
                handoff[out.request_id] = out.kv_transfer_params
    assert all(v and v["remote_block_ids"] for v in handoff.values())
    for i, p in enumerate(prompts):
        D.add_request(p, SamplingParams(max_tokens=max_tokens), request_id=f"r{i}", kv_transfer_params=dict(handoff[f"r{i}"]))
    outs = {}
    t0 = time.time()
    while D.has_unfinished and time.time() - t0 < deadline_s:
        for out in D.step():
            outs.setdefault(out.request_id, []).extend(out.new_token_ids)
        P.step()              # lets the producer observe finished_sending and free its blocks
        time.sleep(0.001)
    return outs


@pytest.fixture(autouse=True)
def _reset_hub():
    InProcessHub.reset()
    yield
    InProcessHub.reset()


def _mixed_reference(prompts, max_tokens):
    E = EngineCore(EngineConfig(block_size=16, num_kv_blocks=48, max_model_len=160, device="cpu", seed=0))
    ids = [E.add_request(p, SamplingParams(max_tokens=max_tokens)) for p in prompts]
    outs = E.run_until_done()
    return [outs[i] for i in ids]


def test_pd_matches_single_instance_and_frees_producer_blocks():
    prompts = _prompts()
    want = _mixed_reference(prompts, 8)
    P, D = _engine("kv_producer", "p0"), _engine("kv_consumer", "d0")
    free_before = P.kv.num_free_blocks
    outs = _run_pd(P, D, prompts, 8)
    assert [outs[f"r{i}"] for i in range(len(prompts))] == want
    for _ in range(20):
        P.step()
    assert P.kv.num_free_blocks == free_before and not P.scheduler.pending_free
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 0


def test_dropped_push_request_is_retried_and_duplicate_acks_ignored():
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 5)
    P, D = _engine("kv_producer", "p1"), _engine("kv_consumer", "d1")
    InProcessHub.drop_next = 1
    InProcessHub.duplicate_acks = True
    outs = _run_pd(P, D, prompts, 5)
    assert [outs[f"r{i}"] for i in range(2)] == want


def test_transfer_that_never_completes_falls_back_to_local_prefill():
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 5)
    P = _engine("kv_producer", "p2")
    D = _engine("kv_consumer", "d2", sync_timeout_s=0.6, retries=1, retry_wait_s=0.2)
    InProcessHub.drop_next = 100           # the producer never hears about the requests
    outs = _run_pd(P, D, prompts, 5)
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 2
    assert [outs[f"r{i}"] for i in range(2)] == want
    # the consumer's cancel told the producer that nobody will come for these blocks: they are free again
    for _ in range(50):
        P.step()
        if not P.scheduler.pending_free:
            break
        time.sleep(0.01)
    assert not P.scheduler.pending_free and P.scheduler.kv.num_free_blocks == 47


def test_producer_releases_blocks_that_nobody_asks_for():
    """The client went away after the prefill (or the decode instance died): the hand-over expires, the blocks are
    freed, and a push request that arrives afterwards is refused, so the late consumer prefills the prompt itself."""
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 4)
    P = _engine("kv_producer", "p9")
    conn = P.worker.runner.kv_connector
    conn.handover_ttl_s = 0.3
    handoff = {}
    for i, p in enumerate(prompts):
        P.add_request(p, SamplingParams(max_tokens=1), request_id=f"r{i}", kv_transfer_params={"do_remote_decode": True})
    while P.scheduler.has_unfinished:
        for out in P.step():
            if out.finished:
                handoff[out.request_id] = out.kv_transfer_params
    assert len(P.scheduler.pending_free) == 2 and P.scheduler.kv.num_free_blocks < 47
    t0 = time.time()
    while P.scheduler.pending_free and time.time() - t0 < 5.0:
        P.step()
        time.sleep(0.02)
    assert not P.scheduler.pending_free and P.scheduler.kv.num_free_blocks == 47 and conn.expired_handovers == 2
    D = _engine("kv_consumer", "d9")
    for i, p in enumerate(prompts):
        D.add_request(p, SamplingParams(max_tokens=4), request_id=f"r{i}", kv_transfer_params=dict(handoff[f"r{i}"]))
    outs = {}
    t0 = time.time()
    while D.has_unfinished and time.time() - t0 < 30.0:
        for out in D.step():
            outs.setdefault(out.request_id, []).extend(out.new_token_ids)
        time.sleep(0.001)
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 2
    assert [outs[f"r{i}"] for i in range(2)] == want


def test_unknown_request_is_refused_and_prefilled_locally():
    """A producer that lost its state (restart) answers nack: the consumer must not decode on blocks nobody wrote."""
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 5)
    P, D = _engine("kv_producer", "p3"), _engine("kv_consumer", "d3")
    real = P.worker.runner.kv_connector
    orig = real.expect_pull
    real.expect_pull = lambda rid: None          # the producer "forgets" every hand-over
    outs = _run_pd(P, D, prompts, 5)
    real.expect_pull = orig
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 2
    assert [outs[f"r{i}"] for i in range(2)] == want


def test_late_and_foreign_acks_do_not_complete_a_request():
    from omni_infer_b200.accelerators.pd.connector import ReqMeta, WorkerConnector
    c = WorkerConnector("kv_consumer", "cx", "inproc://cx", sync_timeout_s=0.3, retries=0, retry_wait_s=0.05)
    with c._lock:
        c._inflight["a"] = (ReqMeta("a", [1], [2], "inproc://nobody"), "cx:7")
    c.handle_ack({"op": "ack", "request_id": "a", "attempt": "cx:6"})      # an older attempt
    c.handle_ack({"op": "ack", "request_id": "zzz", "attempt": "cx:7"})    # a stranger
    assert c.get_finished()[1] == set() and "a" in c._inflight
    c.handle_ack({"op": "ack", "request_id": "a", "attempt": "cx:7"})
    assert c.get_finished()[1] == {"a"}


def test_cancel_waits_for_a_running_copy_and_blocks_later_pushes():
    import threading

    from omni_infer_b200.accelerators.pd.connector import WorkerConnector
    prod = WorkerConnector("kv_producer", "px", "inproc://px")
    cons = WorkerConnector("kv_consumer", "cy", "inproc://cy")
    prod.kv_tensors = [torch.zeros(4, 8)]
    cons.kv_tensors = [torch.zeros(4, 8)]
    prod.expect_pull("q")
    with prod._lock:
        prod._copying.add("q")                   # a copy of the request is "running"
    done = []
    th = threading.Thread(target=lambda: (prod.handle_cancel({"op": "cancel", "request_id": "q", "attempt": "cy:1",
                                                              "reply_to": "inproc://cy"}), done.append(1)))
    th.start()
    time.sleep(0.05)
    assert not done and ("q", "cy:1") not in cons._cancel_acked          # confirmation is held back
    with prod._lock:
        prod._copying.discard("q")
    th.join(2)
    assert done and ("q", "cy:1") in cons._cancel_acked
    # the cancelled attempt is never copied, even if its push request arrives afterwards
    prod.kv_tensors[0].fill_(3.0)
    prod.handle_push_request({"op": "push", "request_id": "q", "attempt": "cy:1", "src_blocks": [0], "dst_blocks": [1],
                              "reply_to": "inproc://cy"})
    assert float(cons.kv_tensors[0].sum()) == 0.0


def test_wire_format_is_json_and_needs_a_key_off_loopback():
    from omni_infer_b200.accelerators.pd.connector import TcpTransport, _decode, _encode
    msg = {"op": "push", "request_id": "r", "cache": {"ipc": [bytes(range(64))], "num_blocks": 3}}
    raw = _encode(msg)
    assert raw.startswith(b"{") and _decode(raw) == msg
    with pytest.raises(ValueError):
        TcpTransport("tcp://10.1.2.3:1", None)


def test_tcp_control_channel_keeps_connections_and_reconnects():
    """Messages between two connectors travel over one kept connection per peer; when the peer went away and came
    back (a restart), the next message reconnects by itself."""
    import socket
    import threading
    import time
    from omni_infer_b200.accelerators.pd.connector import TcpTransport

    class Sink:
        def __init__(self):
            self.got, self.ev = [], threading.Event()

        def dispatch(self, msg):
            self.got.append(msg)
            self.ev.set()

    def port():
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        p = s.getsockname()[1]
        s.close()
        return p

    def wait(sink, n):
        for _ in range(200):
            if len(sink.got) >= n:
                return True
            time.sleep(0.01)
        return False

    a_sink, b_sink = Sink(), Sink()
    pa, pb = port(), port()
    a, b = TcpTransport(f"tcp://127.0.0.1:{pa}", a_sink), TcpTransport(f"tcp://127.0.0.1:{pb}", b_sink)
    try:
        for i in range(5):
            assert a.send(f"tcp://127.0.0.1:{pb}", {"op": "push", "request_id": f"r{i}", "blob": bytes([i]) * 8})
        assert wait(b_sink, 5) and sorted(m["request_id"] for m in b_sink.got) == [f"r{i}" for i in range(5)]
        assert b_sink.got[0]["blob"] in [bytes([i]) * 8 for i in range(5)]
        assert len(a._out) == 1                                    # one connection, reused
        assert b.send(f"tcp://127.0.0.1:{pa}", {"op": "ack", "request_id": "r0"}) and wait(a_sink, 1)
        # the peer restarts on the same port: the kept connection is dead, the next send reconnects
        b.close()
        time.sleep(0.05)
        b2_sink = Sink()
        b2 = TcpTransport(f"tcp://127.0.0.1:{pb}", b2_sink)
        try:
            ok = False
            for _ in range(3):          # the first frame after the restart may still go into the dead socket's buffer
                ok = a.send(f"tcp://127.0.0.1:{pb}", {"op": "push", "request_id": "after"}) and wait(b2_sink, 1)
                if ok:
                    break
            assert ok and b2_sink.got[-1]["request_id"] == "after"
        finally:
            b2.close()
        assert not a.send("tcp://127.0.0.1:1", {"op": "push"})     # nobody listens there: reported, not raised
    finally:
        a.close()


def test_request_dropped_during_its_kv_transfer_keeps_its_blocks_until_the_transfer_is_over():
    """A client that disconnects while the decode instance waits for the KV: the blocks must not return to the pool
    while a producer could still write into them.  The transfer is cancelled with the producer, the request then ends
    as aborted with its blocks freed on both sides, and a request that was not dropped is unaffected."""
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 4)
    P = _engine("kv_producer", "p10")
    D = _engine("kv_consumer", "d10", sync_timeout_s=3.0, retries=3, retry_wait_s=0.3)
    handoff = {}
    for i, p in enumerate(prompts):
        P.add_request(p, SamplingParams(max_tokens=1), request_id=f"r{i}", kv_transfer_params={"do_remote_decode": True})
    while P.scheduler.has_unfinished:
        for out in P.step():
            if out.finished:
                handoff[out.request_id] = out.kv_transfer_params
    InProcessHub.drop_next = 1                 # r0's first push request is lost: its transfer is "on the way" for a while
    D.add_request(prompts[0], SamplingParams(max_tokens=4), request_id="r0", kv_transfer_params=dict(handoff["r0"]))
    D.step()
    r0 = D.scheduler.requests["r0"]
    assert r0.status.name == "WAITING_FOR_REMOTE_KVS" and r0.block_ids
    held = list(r0.block_ids)
    D.abort("r0")
    assert not r0.is_finished and r0.block_ids == held and all(D.scheduler.kv.ref[b] == 1 for b in held)
    D.abort("r0")                              # twice is harmless
    D.add_request(prompts[1], SamplingParams(max_tokens=4), request_id="r1", kv_transfer_params=dict(handoff["r1"]))
    outs = {}
    t0 = time.time()
    while (D.has_unfinished or P.scheduler.pending_free) and time.time() - t0 < 20.0:
        for out in D.step():
            outs.setdefault(out.request_id, []).extend(out.new_token_ids)
        P.step()
        time.sleep(0.002)
    assert r0.status.name == "FINISHED_ABORTED" and not r0.block_ids and "r0" not in outs
    assert outs["r1"] == want[1]
    assert D.scheduler.kv.num_free_blocks == 47 and not D.scheduler._aborting
    assert P.scheduler.kv.num_free_blocks == 47 and not P.scheduler.pending_free


def test_deployment_table_limits_who_exchanges_kv(tmp_path, monkeypatch):
    """With a deployment table in force a decode instance asks only listed prefill instances for KV and a prefill
    instance pushes only to listed decode instances; anything else is prefilled locally."""
    from omni_infer_b200.accelerators.pd.topology import Instance, Topology, from_env
    table = tmp_path / "global_topology.json"
    Topology([Instance("prefill-0", "prefill", [0], 9000, 1, host="p11"), Instance("decode-0", "decode", [1], 9100, 2, host="d11")]).save(str(table))
    monkeypatch.setenv("OMNI_TOPOLOGY", str(table))
    assert from_env().control_endpoints("prefill") == {"tcp://p11:1"}
    prompts = _prompts(2)
    want = _mixed_reference(prompts, 4)

    def engines(p_name, d_name):
        InProcessHub.reset()
        P, D = _engine("kv_producer", p_name), _engine("kv_consumer", d_name)
        return P, D

    # (the engines read the table at start; the endpoints of this test are "inproc://<name>", so each case states who
    # is listed)
    # listed on both sides: KV travels
    P, D = engines("p11", "d11")
    assert D.worker.runner.kv_connector.known_producers == {"tcp://p11:1"}        # what the table said
    for eng in (P, D):
        c = eng.worker.runner.kv_connector
        c.known_producers, c.known_consumers = {"inproc://p11"}, {"inproc://d11"}
    outs = _run_pd(P, D, prompts, 4)
    assert [outs[f"r{i}"] for i in range(2)] == want and D.scheduler.stats.get("kv_fallbacks", 0) == 0
    # the decode instance does not know this prefill instance: it asks nothing of it and prefills itself
    P, D = engines("p12", "d12")
    D.worker.runner.kv_connector.known_producers = {"inproc://somebody-else"}
    outs = _run_pd(P, D, prompts, 4)
    assert [outs[f"r{i}"] for i in range(2)] == want
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 2 and D.worker.runner.kv_connector.refused_strangers == 2
    # the prefill instance does not know this decode instance: refused, prefilled locally
    P, D = engines("p13", "d13")
    D.worker.runner.kv_connector.known_producers = {"inproc://p13"}
    P.worker.runner.kv_connector.known_consumers = {"inproc://somebody-else"}
    outs = _run_pd(P, D, prompts, 4)
    assert [outs[f"r{i}"] for i in range(2)] == want
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 2 and P.worker.runner.kv_connector.refused_strangers == 2
    # an unreadable table is not fatal
    table.write_text("{not json")
    assert from_env() is None


@pytest.mark.parametrize("p_kw,d_kw,mtp", [
    (dict(enable_prefix_caching=True), dict(num_step=3), False),
    (dict(enable_chunked_prefill=True, max_num_batched_tokens=24), dict(async_schedule=True), False),
    (dict(enable_prefix_caching=True, enable_chunked_prefill=True, max_num_batched_tokens=32), dict(num_step=2, num_speculative_tokens=1), True),
    (dict(), dict(num_kv_blocks=11, num_speculative_tokens=1), True),
], ids=["prefix+multistep", "chunked+async", "prefix+chunked+mtp+multistep", "mtp+tight-decode-pool"])
def test_pd_with_engine_features_on_both_sides(p_kw, d_kw, mtp):
    """Prefill and decode instances with different engine options (prefix cache and chunked prefill on the prefill side;
    multi-step, drafts, asynchronous scheduling and a KV pool small enough to preempt on the decode side): the tokens
    equal those of one plain instance, and both sides end with every block free."""
    over = {"num_nextn_predict_layers": 1} if mtp else {}
    g = torch.Generator().manual_seed(21)
    shared = torch.randint(0, 1024, (32,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 1024, (int(n),), generator=g).tolist() for n in (5, 11)]
    prompts.append(torch.randint(0, 1024, (40,), generator=g).tolist())
    E = EngineCore(EngineConfig(block_size=16, num_kv_blocks=48, max_model_len=160, device="cpu", seed=0, model_overrides=over))
    ids = [E.add_request(p, SamplingParams(max_tokens=12)) for p in prompts]
    ref = E.run_until_done()
    want = [ref[i] for i in ids]
    P = _engine("kv_producer", "p20", model_overrides=over, **p_kw)
    D = _engine("kv_consumer", "d20", model_overrides=over, **d_kw)
    outs = _run_pd(P, D, prompts, 12)
    assert [outs[f"r{i}"] for i in range(3)] == want
    for _ in range(50):
        P.step()
        if not P.scheduler.pending_free:
            break
        time.sleep(0.01)
    assert not P.scheduler.pending_free
    assert P.scheduler.kv.num_free_blocks == P.scheduler.kv.num_blocks - 1
    assert D.scheduler.kv.num_free_blocks == D.scheduler.kv.num_blocks - 1
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 0
    if d_kw.get("num_kv_blocks"):
        assert D.scheduler.stats["preemptions"] > 0        # a request whose KV came from the prefill side was recomputed here


@pytest.mark.parametrize("prompt_len", [40, 64, 65, 100, 128])
def test_pd_into_a_decode_instance_with_omni_attention(prompt_len):
    """The decode instance keeps, for compressed layers, a 64-token window per request (16 sink + 48 recent).  The
    prefill instance sends full blocks for the full layers and, for the compressed ones, only the tokens the window
    keeps, at the window positions: the decode instance then generates exactly what one Omni-Attention instance that
    prefilled the prompt itself generates."""
    g = torch.Generator().manual_seed(31)
    prompts = [torch.randint(0, 1024, (prompt_len + d,), generator=g).tolist() for d in (0, 3)]
    omni = dict(enable_omni_attn=True, omni_attn_config={"sink": 1, "recent": 3, "pattern": [0, 1]})
    base = dict(block_size=16, num_kv_blocks=64, max_model_len=256, device="cpu", seed=0, max_num_seqs=4)
    E = EngineCore(EngineConfig(**base, **omni))
    ids = [E.add_request(p, SamplingParams(max_tokens=20)) for p in prompts]
    ref = E.run_until_done()
    want = [ref[i] for i in ids]

    def engine(role, name, **kw):
        return EngineCore(EngineConfig(**base, kv_transfer_config={"kv_role": role, "engine_id": name, "endpoint": f"inproc://{name}",
                                                                   "sync_timeout_s": 5.0, "retries": 3, "retry_wait_s": 0.2}, **kw))

    P, D = engine("kv_producer", "p30"), engine("kv_consumer", "d30", **omni)
    conn = D.worker.runner.kv_connector
    assert conn.compressed_idx == [1] and conn.omni_spec.capacity_tokens == 64
    outs = _run_pd(P, D, prompts, 20)
    assert [outs[f"r{i}"] for i in range(2)] == want
    assert D.scheduler.stats.get("kv_fallbacks", 0) == 0                     # the KV really came from the prefill instance
    assert len(D.kv.window_free) == 4 * 4 and D.kv.num_free_blocks == 63


def test_the_reused_prefill_token_counts_towards_the_stop_conditions():
    """The decode instance takes its first token from the prefill instance.  That token is an output token like any
    other: a request with ``max_tokens = 1``, or one whose first token is a stop id, ends with it instead of decoding
    one more."""
    prompts = _prompts(2, 30, seed=8)
    want = _mixed_reference(prompts, 5)
    P, D = _engine("kv_producer", "p40"), _engine("kv_consumer", "d40")
    handoff = {}
    for i, p in enumerate(prompts):
        P.add_request(p, SamplingParams(max_tokens=1), request_id=f"r{i}", kv_transfer_params={"do_remote_decode": True})
    while P.scheduler.has_unfinished:
        for out in P.step():
            if out.finished:
                handoff[out.request_id] = out.kv_transfer_params
    D.add_request(prompts[0], SamplingParams(max_tokens=1), request_id="r0", kv_transfer_params=dict(handoff["r0"]))
    D.add_request(prompts[1], SamplingParams(max_tokens=5, stop_token_ids=(want[1][0],)), request_id="r1",
                  kv_transfer_params=dict(handoff["r1"]))
    outs, reasons = {}, {}
    t0 = time.time()
    while (D.has_unfinished or P.scheduler.pending_free) and time.time() - t0 < 20:
        for out in D.step():
            outs.setdefault(out.request_id, []).extend(out.new_token_ids)
            if out.finished:
                reasons[out.request_id] = out.finish_reason
        P.step()
        time.sleep(0.001)
    assert outs == {"r0": want[0][:1], "r1": want[1][:1]}
    assert reasons == {"r0": "length", "r1": "stop"}
    assert D.scheduler.kv.num_free_blocks == 47 and P.scheduler.kv.num_free_blocks == 47
