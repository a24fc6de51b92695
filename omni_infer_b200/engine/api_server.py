"""OpenAI-compatible HTTP front end over one engine (one API server + one engine core per data-parallel rank, as
the reference arranges with its scale-out patch).

  POST /v1/completions, /v1/chat/completions   streaming (SSE) or not
  GET  /health, /metrics                        liveness and Prometheus text
  POST /start_profile, /stop_profile            torch profiler on the worker

Behaviour carried over from the reference's engine patches:
  * every stream chunk carries ``prompt_num_token`` / ``output_num_token`` and ``usage.total_tokens`` so the proxy's
    body filters can track decode load (num_token_for_proxy.patch)
  * a request with ``kv_transfer_params.do_remote_decode`` (sent by the proxy with max_tokens = 1) answers with the
    ``kv_transfer_params`` for the decode instance, including ``prompt_token_ids`` and the ``prefilled_token`` so the
    decode side neither tokenises again nor recomputes the first token (tokenizer_proc_pool.patch,
    patch_support_prefilled_token_skip_tokenize.patch)
  * long prompts are tokenised in the process pool (engine/tokenizer_pool.py)
  * keep-alive timeout 120 s."""
from __future__ import annotations

import json
import logging
import queue
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

from .engine_core import EngineConfig, EngineCore
from .request import SamplingParams
from .tokenizer_pool import TokenizerPool
from ..utils import timeline

logger = logging.getLogger("omni_infer_b200.api")


class AsyncEngine:
    """Engine loop on its own thread; per-request output queues."""

    def __init__(self, engine: EngineCore):
        self.engine = engine
        self.queues: dict = {}
        self.lock = threading.Lock()
        self.inbox: queue.Queue = queue.Queue()
        self._stop = False
        self.stats = {"requests": 0, "tokens": 0, "started": time.time(), "failed_steps": 0}
        self.failed_in_a_row = 0          # engine steps that raised, since the last one that did not
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def submit(self, prompt_ids, sampling, request_id, kv_transfer_params=None, priority: int = 0) -> Optional[queue.Queue]:
        q: queue.Queue = queue.Queue()
        with self.lock:
            if request_id in self.queues:
                return None
            self.queues[request_id] = q
        self.inbox.put((prompt_ids, sampling, request_id, kv_transfer_params, priority))
        self.stats["requests"] += 1
        return q

    def abort(self, request_id):
        """Called by the request's own handler once it has stopped reading: an aborted request produces no finished
        output, so its queue is dropped here and not by the loop."""
        with self.lock:
            self.queues.pop(request_id, None)
        self.inbox.put(("abort", request_id))

    def _fail(self, request_id):
        with self.lock:
            q = self.queues.pop(request_id, None)
        if q is not None:
            q.put(None)

    UNHEALTHY_AFTER = 3

    @property
    def healthy(self) -> bool:
        """False after several engine steps in a row have failed (a lost device or peer): ``/health`` then answers 503
        so that the proxy takes this instance out of rotation instead of feeding it requests that will fail."""
        return self.failed_in_a_row < self.UNHEALTHY_AFTER

    def _loop(self):
        eng = self.engine
        held: list = []
        while not self._stop:
            try:
                while True:
                    item = self.inbox.get_nowait() if (eng.has_unfinished or eng._world > 1) else self.inbox.get(timeout=0.05)
                    if item[0] == "abort":
                        eng.abort(item[1])
                    elif item[2] in eng.scheduler.requests and not eng.scheduler.requests[item[2]].is_finished:
                        # the id of a request that has been dropped but takes part in the round being executed (a client
                        # that retries at once under its old id): the new one is taken in after that round
                        if item[2] in eng._deferred_aborts:
                            held.append(item)
                        else:
                            self._fail(item[2])
                    else:
                        try:
                            eng.add_request(item[0], item[1], item[2], item[3], priority=item[4])
                        except Exception:  # noqa: BLE001  (one request the engine refuses must not end the serving thread)
                            logger.exception("the engine refused request %s", item[2])
                            self._fail(item[2])
            except queue.Empty:
                pass
            for item in held:
                self.inbox.put(item)
            held = []
            if not eng.has_unfinished:
                if eng._world == 1:
                    if not eng.scheduler.pending_free:
                        continue
                    # a prefill instance that has gone idle still holds the blocks of its last hand-overs: it keeps
                    # stepping (slowly) so that they are released when the decode side has fetched them or their time is up
                    time.sleep(0.02)
                # several data-parallel ranks share the expert-parallel exchanges: an idle rank keeps stepping (dummy
                # batches) so that busy peers never wait for it; when the whole group was idle it paces itself
                elif not eng.peers_busy:
                    time.sleep(0.002)
            try:
                outs = eng.step()
            except Exception as e:  # noqa: BLE001  (a failed step must not kill the serving thread)
                logger.exception("engine step failed: %s", e)
                self.stats["failed_steps"] += 1
                self.failed_in_a_row += 1
                with self.lock:
                    failed = list(self.queues.items())
                    self.queues.clear()
                for rid, q in failed:
                    # out of the scheduler too: the same batch must not be run (and fail) again for ever
                    try:
                        eng.abort(rid)
                    except Exception:  # noqa: BLE001
                        logger.exception("could not drop %s after the failed step", rid)
                    q.put(None)
                if self.failed_in_a_row >= self.UNHEALTHY_AFTER:
                    time.sleep(0.2)         # nothing works: do not spin
                continue
            self.failed_in_a_row = 0
            for o in outs:
                self.stats["tokens"] += len(o.new_token_ids)
                with self.lock:
                    q = self.queues.get(o.request_id)
                    if o.finished:
                        self.queues.pop(o.request_id, None)
                if q is not None:
                    q.put(o)

    def stop(self):
        self._stop = True
        try:
            self.engine.save_state()
        except Exception:                      # shutting down: a state file that cannot be written must not hang it
            logging.getLogger("omni_infer_b200.api_server").exception("could not write the state directory")


class _QuietServer(ThreadingHTTPServer):
    """A client that hangs up between requests is routine for a server behind a proxy: one log line, not a stack trace."""
    daemon_threads = True
    request_queue_size = 128

    def handle_error(self, request, client_address):
        import sys
        e = sys.exc_info()[1]
        if isinstance(e, (ConnectionError, TimeoutError)):
            logger.debug("client %s went away: %s", client_address, e)
            return
        super().handle_error(request, client_address)


def _make_parsers(reasoning_parser: Optional[str], tool_call_parser: Optional[str]):
    """Parser objects for the chat endpoint by name (the host engine's ``--reasoning-parser`` / ``--tool-call-parser``)."""
    known_r, known_t = {}, {}
    from ..models.pangu.reasoning import PanguReasoningParser
    from ..models.pangu.tool_parser import PanguToolParser
    known_r["pangu"], known_t["pangu"] = PanguReasoningParser, PanguToolParser
    if reasoning_parser and reasoning_parser not in known_r:
        raise ValueError(f"unknown reasoning parser {reasoning_parser!r} (known: {sorted(known_r)})")
    if tool_call_parser and tool_call_parser not in known_t:
        raise ValueError(f"unknown tool-call parser {tool_call_parser!r} (known: {sorted(known_t)})")
    return (known_r[reasoning_parser]() if reasoning_parser else None, known_t[tool_call_parser]() if tool_call_parser else None)


def make_handler(aeng: AsyncEngine, tok: TokenizerPool, model_name: str, reasoning=None, tools=None):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        timeout = 120           # keep-alive

        def log_message(self, *a):
            pass

        def _json(self, code, obj):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def _client_gone(self) -> bool:
            """True when the peer has closed its side (no request is pipelined behind a pending one here, so readable +
            zero bytes means end of stream)."""
            import select
            import socket
            try:
                r, _, _ = select.select([self.connection], [], [], 0)
                if not r:
                    return False
                return self.connection.recv(1, socket.MSG_PEEK | socket.MSG_DONTWAIT) == b""
            except (BlockingIOError, InterruptedError):
                return False
            except OSError:
                return True

        def do_GET(self):
            if self.path == "/health":
                if not aeng.healthy:
                    return self._json(503, {"status": "engine steps are failing", "failed_steps": aeng.stats["failed_steps"]})
                return self._json(200, {"status": "ok"})
            if self.path == "/metrics":
                s, e = aeng.stats, aeng.engine
                text = (f"omni_requests_total {s['requests']}\nomni_generated_tokens_total {s['tokens']}\n"
                        f"omni_running_requests {e.scheduler.num_running}\nomni_waiting_requests {e.scheduler.num_waiting}\n"
                        f"omni_kv_cache_usage {e.kv.usage:.4f}\nomni_preemptions_total {e.scheduler.stats['preemptions']}\n"
                        f"omni_failed_steps_total {s['failed_steps']}\nomni_engine_healthy {int(aeng.healthy)}\n"
                        f"omni_engine_steps_total {e.metrics['steps']}\n").encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(text)))
                self.end_headers()
                self.wfile.write(text)
                return
            if self.path == "/v1/models":
                return self._json(200, {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "omni_infer_b200",
                                                                    "max_model_len": aeng.engine.cfg.max_model_len}]})
            if self.path == "/version":
                from .. import __version__
                return self._json(200, {"version": __version__})
            self._json(404, {"error": "not found"})

        def send_response(self, code, message=None):
            self._answered = True
            super().send_response(code, message)

        def do_POST(self):
            """A fault in the handler itself is answered with a 500 when no answer has been started (a client must not be
            left with a connection that closes without a word), and logged either way."""
            self._answered = False
            try:
                return self._post()
            except (ConnectionError, TimeoutError):
                raise
            except Exception as e:  # noqa: BLE001
                logger.exception("request handler failed: %s", e)
                self.close_connection = True
                if not self._answered:
                    try:
                        self._json(500, {"error": f"internal error: {type(e).__name__}"})
                    except OSError:
                        pass

        def _post(self):
            try:
                n = int(self.headers.get("Content-Length", "0"))
                if n < 0:
                    raise ValueError
            except ValueError:
                self.close_connection = True            # where the body ends is unknown: nothing more is read here
                return self._json(400, {"error": "bad Content-Length"})
            try:
                body = json.loads(self.rfile.read(n) or b"{}")
            except (json.JSONDecodeError, UnicodeDecodeError):
                return self._json(400, {"error": "invalid JSON"})
            if not isinstance(body, dict):
                return self._json(400, {"error": "the request body must be a JSON object"})
            if self.path == "/tokenize":
                text = body.get("prompt")
                if not isinstance(text, str):
                    return self._json(400, {"error": "prompt must be a string"})
                ids = tok.encode(text)
                return self._json(200, {"tokens": ids, "count": len(ids), "max_model_len": aeng.engine.cfg.max_model_len})
            if self.path == "/detokenize":
                ids = body.get("tokens")
                if not isinstance(ids, list) or not all(isinstance(t, int) and not isinstance(t, bool) for t in ids):
                    return self._json(400, {"error": "tokens must be a list of integers"})
                return self._json(200, {"prompt": tok.decode(ids)})
            if self.path in ("/start_profile", "/stop_profile"):
                aeng.engine.worker.profile(self.path == "/start_profile")
                return self._json(200, {"status": "ok"})
            chat = self.path == "/v1/chat/completions"
            if not chat and self.path != "/v1/completions":
                return self._json(404, {"error": "not found"})
            kvp = body.get("kv_transfer_params")
            if kvp is not None and not isinstance(kvp, dict):
                return self._json(400, {"error": "kv_transfer_params must be an object"})
            if (body.get("n") or 1) != 1 or body.get("logprobs") or body.get("top_logprobs"):
                return self._json(400, {"error": "n > 1 and logprobs are not supported"})

            def token_list(v):
                return isinstance(v, list) and all(isinstance(t, int) and not isinstance(t, bool) for t in v)
            # decode instance: reuse the prompt ids produced by the prefill instance
            if kvp and kvp.get("prompt_token_ids"):
                if not token_list(kvp["prompt_token_ids"]):
                    return self._json(400, {"error": "kv_transfer_params.prompt_token_ids must be a list of integers"})
                ids = list(kvp["prompt_token_ids"])
            elif chat:
                msgs = body.get("messages")
                if not isinstance(msgs, list) or not all(isinstance(m, dict) for m in msgs):
                    return self._json(400, {"error": "messages must be a list of objects"})
                # content given as a list of parts: the text parts, joined
                msgs = [dict(m, content="".join(str(c.get("text", "")) for c in m["content"] if isinstance(c, dict)))
                        if isinstance(m.get("content"), list) else m for m in msgs]
                ids = tok.encode(tok.tokenizer.apply_chat_template(msgs, add_generation_prompt=True)
                                 if hasattr(tok.tokenizer, "apply_chat_template") else str(msgs))
            else:
                p = body.get("prompt")
                if isinstance(p, list) and len(p) == 1 and isinstance(p[0], (str, list)):
                    p = p[0]                            # a batch of one
                if token_list(p):
                    ids = list(p)                       # token ids as they are (an empty list is an empty prompt)
                elif isinstance(p, str):
                    ids = tok.encode(p)
                else:
                    return self._json(400, {"error": "prompt must be a string or a list of token ids (one prompt per request)"})
            vocab = getattr(getattr(aeng.engine, "model_cfg", None), "vocab_size", None)
            if vocab is not None and ids and (min(ids) < 0 or max(ids) >= vocab):
                # the embedding lookup trusts its indices: an id outside the table must never reach the device
                return self._json(400, {"error": f"token ids must lie in [0, {vocab})"})
            try:
                want = body.get("max_tokens") if body.get("max_tokens") is not None else body.get("max_completion_tokens")
                if isinstance(want, bool) or (want is not None and int(want) != want):
                    raise ValueError("max_tokens must be an integer")
                sp = SamplingParams(max_tokens=16 if want is None else int(want),
                                    temperature=float(body.get("temperature", 0.0) or 0.0), top_k=int(body.get("top_k", 0) or 0),
                                    top_p=float(body.get("top_p", 1.0) or 1.0), ignore_eos=bool(body.get("ignore_eos", False)),
                                    stop_token_ids=tuple(int(t) for t in (body.get("stop_token_ids") or ())),
                                    seed=None if body.get("seed") is None else int(body["seed"]),
                                    repetition_penalty=float(body.get("repetition_penalty", 1.0) or 1.0),
                                    presence_penalty=float(body.get("presence_penalty", 0.0) or 0.0),
                                    frequency_penalty=float(body.get("frequency_penalty", 0.0) or 0.0))
                stop = body.get("stop") or []
                stop = [stop] if isinstance(stop, str) else [str(x) for x in stop]
                if sp.repetition_penalty <= 0:
                    raise ValueError("repetition_penalty must be positive")
                if sp.max_tokens < 1 or sp.temperature < 0 or not 0 < sp.top_p <= 1 or sp.top_k < 0:
                    raise ValueError("max_tokens >= 1, temperature >= 0, 0 < top_p <= 1 and top_k >= 0 are required")
            except (TypeError, ValueError) as e:
                return self._json(400, {"error": f"invalid sampling parameters: {e}"})
            if not ids:
                return self._json(400, {"error": "empty prompt"})
            limit = aeng.engine.cfg.max_model_len
            if len(ids) >= limit:
                return self._json(400, {"error": f"the prompt has {len(ids)} tokens; this model's context holds {limit} "
                                                 f"including the completion"})
            rid = self.headers.get("X-Request-Id") or ("cmpl-" + uuid.uuid4().hex)
            timeline.emit("Get request in api server", rid, role=aeng.engine.role)
            try:
                priority = int(body.get("priority", 0) or 0)       # used by the priority scheduling policy
            except (TypeError, ValueError):
                return self._json(400, {"error": "priority must be an integer"})
            q = aeng.submit(ids, sp, rid, kvp, priority)
            if q is None:       # a client-chosen id that is still in flight: answering on the first one's queue would mix them
                return self._json(409, {"error": f"request id {rid!r} is already in flight"})
            stream = bool(body.get("stream", False))
            created = int(time.time())
            n_prompt, out_ids, final = len(ids), [], None
            sent_text, final_text, final_reason = "", None, None
            saw_tool_call, content_seen = False, ""

            def chunk_obj(text, finish):
                usage = {"prompt_tokens": n_prompt, "completion_tokens": len(out_ids), "total_tokens": n_prompt + len(out_ids)}
                choice = ({"index": 0, "delta": {"content": text}, "finish_reason": finish} if chat
                          else {"index": 0, "text": text, "finish_reason": finish})
                return {"id": rid, "object": "chat.completion.chunk" if chat else "text_completion", "created": created,
                        "model": model_name, "choices": [choice], "usage": usage, "prompt_num_token": n_prompt,
                        "output_num_token": len(out_ids)}

            if stream:
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self.end_headers()
            try:
                last_output = last_probe = time.monotonic()
                while True:
                    now = time.monotonic()
                    if now - last_probe >= 0.5:           # also while outputs keep coming (a non-streaming reply
                        last_probe = now                  # writes nothing until the end)
                        if self._client_gone():
                            raise BrokenPipeError("the client closed the connection")
                    try:
                        o = q.get(timeout=0.5)
                    except queue.Empty:
                        if time.monotonic() - last_output >= 600:
                            raise
                        continue
                    last_output = time.monotonic()
                    if o is None:
                        raise RuntimeError("engine failure")
                    if o.finished and o.finish_reason == "ignored":
                        raise RuntimeError("the request does not fit this instance (prompt longer than the context or the KV pool)")
                    if not out_ids and o.new_token_ids:
                        timeline.emit("First token out of api server", rid, role=aeng.engine.role)
                    out_ids += o.new_token_ids
                    stopped = None
                    if stop and o.new_token_ids:
                        # stop strings are matched on the text so far (they may straddle tokens); the text ends before
                        # the first one and the request is dropped from the engine
                        text_so_far = tok.decode(out_ids)
                        cuts = [text_so_far.find(x) for x in stop if x and x in text_so_far]
                        if cuts:
                            stopped = text_so_far[:min(cuts)]
                    if stopped is not None:
                        aeng.abort(rid)
                        if stream:
                            tail = stopped[len(sent_text):] if stopped.startswith(sent_text) else ""
                            self.wfile.write(("data: " + json.dumps(chunk_obj(tail, "stop")) + "\n\n").encode())
                            self.wfile.flush()
                        final = o
                        final_text, final_reason = stopped, "stop"
                        break
                    if stream and (o.new_token_ids or o.finished):
                        # incremental detokenisation: what the whole output reads as now, minus what was sent; a
                        # character whose bytes have not all arrived yet is held back until it is complete
                        full = tok.decode(out_ids)
                        stable = full if o.finished else full.rstrip("\ufffd")
                        if stop and not o.finished:
                            # the end of the text may be the beginning of a stop string: not sent until that is settled
                            hold = max((n for x in stop for n in range(1, len(x)) if stable.endswith(x[:n])), default=0)
                            stable = stable[:len(stable) - hold]
                        piece = stable[len(sent_text):] if stable.startswith(sent_text) else tok.decode(o.new_token_ids)
                        obj = chunk_obj(piece, o.finish_reason if o.finished else None)
                        if chat and (reasoning is not None or tools is not None):
                            # the delta is split into reasoning / content / tool calls; markers never reach the client
                            delta = {"content": piece} if piece else {}
                            if reasoning is not None:
                                delta = reasoning.extract_reasoning_content_streaming(sent_text, piece) or {}
                            if tools is not None and delta.get("content"):
                                c = delta.pop("content")
                                t = tools.extract_tool_calls_streaming(content_seen, c) or {}
                                content_seen += c             # what the tool parser has been shown so far
                                delta.update(t)
                                if t.get("tool_calls"):
                                    saw_tool_call = True
                            obj["choices"][0]["delta"] = delta
                            if o.finished and saw_tool_call:
                                obj["choices"][0]["finish_reason"] = "tool_calls"
                        sent_text += piece
                        self.wfile.write(("data: " + json.dumps(obj) + "\n\n").encode())
                        self.wfile.flush()
                    if o.finished:
                        final = o
                        break
            except (BrokenPipeError, ConnectionResetError):
                aeng.abort(rid)
                return
            except (queue.Empty, RuntimeError) as e:
                aeng.abort(rid)
                if not stream:
                    return self._json(500, {"error": str(e) or "timeout"})
                return
            timeline.emit("Finish response in api server", rid, role=aeng.engine.role)
            if stream:
                opts = body.get("stream_options")
                if isinstance(opts, dict) and opts.get("include_usage"):
                    # the closing chunk load generators count tokens from: no choices, the totals of the request
                    last = chunk_obj("", None)
                    last["choices"] = []
                    self.wfile.write(("data: " + json.dumps(last) + "\n\n").encode())
                self.wfile.write(b"data: [DONE]\n\n")
                self.wfile.flush()
                self.close_connection = True
                return
            text = tok.decode(out_ids) if final_text is None else final_text
            reason = final_reason or final.finish_reason
            resp = chunk_obj(text, reason)
            resp["object"] = "chat.completion" if chat else "text_completion"
            if chat:
                message = {"role": "assistant", "content": text}
                if reasoning is not None:
                    message["reasoning_content"], message["content"] = reasoning.extract_reasoning_content(text)
                if tools is not None and message["content"]:
                    ex = tools.extract_tool_calls(message["content"])
                    if ex.tools_called:
                        message["content"], message["tool_calls"] = ex.content, [c.to_dict() for c in ex.tool_calls]
                        reason = "tool_calls"
                resp["choices"][0] = {"index": 0, "message": message, "finish_reason": reason}
            if final.kv_transfer_params:
                resp["kv_transfer_params"] = final.kv_transfer_params
            try:
                self._json(200, resp)
            except (BrokenPipeError, ConnectionResetError):
                self.close_connection = True          # the client left just before the answer: nothing to tell anybody

    return Handler


def serve(engine_cfg: EngineConfig, host: str = "0.0.0.0", port: int = 8000, tokenizer: Optional[str] = None,
          model_cfg=None, block: bool = True, reasoning_parser: Optional[str] = None, tool_call_parser: Optional[str] = None):
    reasoning, tools = _make_parsers(reasoning_parser, tool_call_parser)
    engine = EngineCore(engine_cfg, model_cfg=model_cfg)
    aeng = AsyncEngine(engine)
    tok = TokenizerPool(tokenizer, vocab_size=engine.model_cfg.vocab_size)
    srv = _QuietServer((host, port), make_handler(aeng, tok, engine.model_cfg.name or engine_cfg.model, reasoning, tools))
    srv.daemon_threads = True
    if block:
        try:
            srv.serve_forever()
        finally:
            aeng.stop()
            tok.shutdown()
        return None
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, aeng


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="OpenAI-compatible API server over one engine")
    ap.add_argument("--model", default="tiny-deepseek-v3")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--block-size", type=int, default=128)
    ap.add_argument("--num-kv-blocks", type=int, default=0)
    ap.add_argument("--num-speculative-tokens", type=int, default=0)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--data-parallel-rank", type=int, default=0)
    ap.add_argument("--kv-transfer-config", default=None, help="JSON")
    ap.add_argument("--additional-config", default=None, help="JSON")
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--model-overrides", default=None, help="JSON of model-config fields to override (e.g. fewer layers)")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--enable-chunked-prefill", action="store_true")
    ap.add_argument("--scheduling-policy", default="fcfs", choices=["fcfs", "priority"])
    ap.add_argument("--reasoning-parser", default=None, help="split chat answers into reasoning and content (pangu)")
    ap.add_argument("--tool-call-parser", default=None, help="turn tool-call blocks of chat answers into tool_calls (pangu)")
    ap.add_argument("--enable-auto-tool-choice", action="store_true", help="accepted for compatibility: tool calls are parsed whenever a parser is set")
    a = ap.parse_args(argv)
    cfg = EngineConfig(model=a.model, device=a.device, max_num_seqs=a.max_num_seqs, max_model_len=a.max_model_len,
                       max_num_batched_tokens=a.max_num_batched_tokens, block_size=a.block_size, num_kv_blocks=a.num_kv_blocks,
                       num_speculative_tokens=a.num_speculative_tokens, tp_size=a.tensor_parallel_size,
                       enforce_eager=a.enforce_eager, gpu_memory_utilization=a.gpu_memory_utilization,
                       enable_chunked_prefill=a.enable_chunked_prefill, scheduling_policy=a.scheduling_policy,
                       model_overrides=json.loads(a.model_overrides) if a.model_overrides else {},
                       kv_transfer_config=json.loads(a.kv_transfer_config) if a.kv_transfer_config else None)
    if a.additional_config:
        from ..adaptors.vllm.platform import ConfigUpdater
        ConfigUpdater.update_engine_config(cfg, json.loads(a.additional_config))
    serve(cfg, a.host, a.port, a.tokenizer, reasoning_parser=a.reasoning_parser, tool_call_parser=a.tool_call_parser)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
