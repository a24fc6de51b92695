"""Prefill/decode disaggregation connector (reference: LLMDataDistConnector,
omni/accelerators/pd/llmdatadist_connector_v1.py:87-728, and its transfer manager llmdatadist_manager.py:132-482).

Roles
  * ``kv_producer`` (prefill instance): a request that finishes its single prefill token hands
    ``kv_transfer_params = {remote_block_ids, remote_engine_id, remote_host, spec_token_ids, prompt_token_ids,
    prefilled_token}`` back to the client (the proxy splices it into the decode request) and keeps its blocks until
    the decode side has them.
  * ``kv_consumer`` (decode instance): the scheduler reserves local blocks for the whole prompt
    (``get_num_new_matched_tokens`` -> asynchronous load), the worker side asks the producer to push the blocks
    into its paged cache, and the request leaves WAITING_FOR_REMOTE_KVS when the push is acknowledged.

Transfer: the producer copies blocks into the consumer's cache (NVLink peer memory on GPUs, csrc/kernels/kv_push.cu;
index copy on CPU).  Control messages travel over a pluggable transport: an in-process hub (tests, CPU mock, both
engines in one process) or TCP (``multiprocessing.connection``) between processes, where the consumer registers
the CUDA IPC handles of its cache tensors on first contact.

Robustness: a push request is retried ``retries`` times ``retry_wait_s`` apart and abandoned after
``sync_timeout_s`` (reference: 3 x 2 s, 20 s); an abandoned request is reported in ``failed_recving`` and the
scheduler falls back to prefilling it locally.  Every push carries an attempt id: only the acknowledgement of the
attempt being waited for counts, a producer that does not know the request answers ``nack`` (local prefill at once,
never a decode on blocks nobody wrote), and a consumer that gives up sends ``cancel`` and frees the blocks only after
the producer confirmed that nothing of that attempt is being written any more.  The producer in turn does not keep a
handed-over request's blocks for ever: it releases them when the consumer cancels or is refused (that request is
prefilled on the decode side, the blocks are of no use any more) and when nobody has asked for them within
``handover_ttl_s`` (the client went away, the decode instance died); a push that arrives later is answered ``nack``."""
from __future__ import annotations

import logging
import threading
import time
from dataclasses import dataclass, field
from typing import Optional

import torch

from .kv_push import PeerCacheView, flatten_cache, push_blocks_cuda, push_blocks_torch

logger = logging.getLogger("omni_infer_b200.pd")


@dataclass
class ReqMeta:
    request_id: str
    local_block_ids: list
    remote_block_ids: list
    remote_host: str
    remote_engine_id: str = ""
    # Omni-Attention on the decode instance: the request's window blocks for the compressed layers and what decides
    # which prompt tokens go where in them
    window_block_ids: list = field(default_factory=list)
    prompt_len: int = 0


@dataclass
class ConnectorMetadata:
    requests: list = field(default_factory=list)


# ------------------------------------------------------------------------------------------------ transports
class InProcessHub:
    """Endpoint registry for engines that live in one process.  Fault injection for tests: ``drop_next`` swallows
    that many push requests, ``duplicate_acks`` delivers every acknowledgement twice."""
    endpoints: dict = {}
    drop_next: int = 0
    duplicate_acks: bool = False
    lock = threading.Lock()

    @classmethod
    def reset(cls):
        cls.endpoints, cls.drop_next, cls.duplicate_acks = {}, 0, False

    @classmethod
    def register(cls, endpoint: str, worker) -> None:
        cls.endpoints[endpoint] = worker

    @classmethod
    def send_push_request(cls, endpoint: str, msg: dict) -> bool:
        with cls.lock:
            if cls.drop_next > 0:
                cls.drop_next -= 1
                return True            # the message is lost on the way: the sender cannot tell
        w = cls.endpoints.get(endpoint)
        if w is None:
            return False
        threading.Thread(target=w.handle_push_request, args=(msg,), daemon=True).start()
        return True

    @classmethod
    def send_ack(cls, endpoint: str, msg: dict) -> None:
        w = cls.endpoints.get(endpoint)
        if w is not None:
            w.dispatch(msg)
            if cls.duplicate_acks and msg.get("op") == "ack":
                w.dispatch(msg)

    @classmethod
    def send_cancel(cls, endpoint: str, msg: dict) -> bool:
        w = cls.endpoints.get(endpoint)
        if w is None:
            return False
        threading.Thread(target=w.dispatch, args=(msg,), daemon=True).start()
        return True


def _authkey(key=None) -> bytes:
    """Shared secret of the control channel: the ``authkey`` of the kv-transfer config, else ``OMNI_KV_AUTHKEY``.
    Without one the channel only accepts loopback endpoints."""
    import os
    k = key or os.environ.get("OMNI_KV_AUTHKEY", "")
    return k.encode() if isinstance(k, str) else bytes(k)


def _encode(msg: dict) -> bytes:
    """Wire format: one JSON document per connection (bytes values, the CUDA IPC handles, as base64)."""
    import base64
    import json

    def conv(o):
        if isinstance(o, (bytes, bytearray)):
            return {"__b64__": base64.b64encode(bytes(o)).decode()}
        if isinstance(o, dict):
            return {k: conv(v) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return [conv(v) for v in o]
        return o
    return json.dumps(conv(msg)).encode()


def _decode(raw: bytes) -> dict:
    import base64
    import json

    def conv(o):
        if isinstance(o, dict):
            if set(o) == {"__b64__"}:
                return base64.b64decode(o["__b64__"])
            return {k: conv(v) for k, v in o.items()}
        if isinstance(o, list):
            return [conv(v) for v in o]
        return o
    return conv(json.loads(raw.decode()))


class TcpTransport:
    """Control channel between processes.  Every worker connector listens on its endpoint.  A message is one JSON
    document sent as a byte frame (nothing is unpickled); the connection handshake uses the configured key.
    Messages: push / cancel consumer -> producer, ack / nack / cancel_ack producer -> consumer."""

    def __init__(self, endpoint: str, worker, authkey=None):
        from multiprocessing.connection import Listener
        host, port = endpoint.replace("tcp://", "").rsplit(":", 1)
        self.key = _authkey(authkey)
        if not self.key and host not in ("127.0.0.1", "localhost", "::1"):
            raise ValueError("a kv-transfer endpoint that is not loopback needs an authkey (config 'authkey' or OMNI_KV_AUTHKEY)")
        self.key = self.key or b"omni-pd-loopback"
        self._addr = (host, int(port))
        self.listener = Listener(self._addr, authkey=self.key)
        self.worker = worker
        self._stop = False
        self._out: dict = {}                  # endpoint -> open connection to that peer
        self._out_lock = threading.Lock()
        threading.Thread(target=self._serve, daemon=True).start()

    def _serve(self):
        while not self._stop:
            try:
                conn = self.listener.accept()
            except OSError:
                return
            except Exception:  # noqa: BLE001  (failed handshake of a stranger, or the wake-up connection of close())
                if self._stop:
                    return
                continue
            threading.Thread(target=self._handle, args=(conn,), daemon=True).start()

    def _handle(self, conn):
        # a peer keeps its connection open and sends one frame per message (the handshake of a new connection costs
        # two round trips, which would sit on every request's time to first token)
        try:
            while not self._stop:
                try:
                    raw = conn.recv_bytes(1 << 22)
                except (EOFError, OSError):
                    return
                # one thread per message, as before: a cancel must be able to overtake the copy of a push
                threading.Thread(target=self._dispatch, args=(raw,), daemon=True).start()
        finally:
            conn.close()

    def _dispatch(self, raw: bytes) -> None:
        try:
            self.worker.dispatch(_decode(raw))
        except (ValueError, KeyError) as e:
            logger.warning("kv control message dropped: %s: %s", type(e).__name__, e)

    def _connection(self, endpoint: str):
        from multiprocessing.connection import Client
        c = self._out.get(endpoint)
        if c is None:
            host, port = endpoint.replace("tcp://", "").rsplit(":", 1)
            c = Client((host, int(port)), authkey=self.key)
            self._out[endpoint] = c
        return c

    def send(self, endpoint: str, msg: dict) -> bool:
        frame = _encode(msg)
        with self._out_lock:
            for attempt in range(2):            # a cached connection may have been closed by the peer: reconnect once
                try:
                    self._connection(endpoint).send_bytes(frame)
                    return True
                except Exception:  # noqa: BLE001
                    c = self._out.pop(endpoint, None)
                    if c is not None:
                        try:
                            c.close()
                        except OSError:
                            pass
            return False

    def close(self):
        self._stop = True
        # the accept thread sits in accept(): closing the socket under it would leave the port bound until it returns,
        # so wake it with a connection of our own first
        try:
            import socket
            socket.create_connection(self._addr, timeout=0.5).close()
        except OSError:
            pass
        self.listener.close()
        with self._out_lock:
            for c in self._out.values():
                try:
                    c.close()
                except OSError:
                    pass
            self._out.clear()


# ------------------------------------------------------------------------------------------------ scheduler side
class SchedulerConnector:
    def __init__(self, kv_role: str, engine_id: str, endpoint: str, block_size: int, num_speculative_tokens: int = 0,
                 worker=None):
        self.kv_role, self.engine_id, self.endpoint, self.block_size = kv_role, engine_id, endpoint, block_size
        self.num_spec = num_speculative_tokens
        self.worker = worker                  # same-process worker connector (fast path delivery)
        self._pending: list = []

    @property
    def is_producer(self) -> bool:
        return self.kv_role in ("kv_producer", "kv_both")

    @property
    def is_consumer(self) -> bool:
        return self.kv_role in ("kv_consumer", "kv_both")

    # -- consumer
    def get_num_new_matched_tokens(self, req, num_computed_tokens: int):
        """External tokens = the prompt rounded up to whole blocks, loaded asynchronously."""
        p = req.kv_transfer_params or {}
        if not (self.is_consumer and p.get("do_remote_prefill") and p.get("remote_block_ids")):
            return 0, False
        n = len(req.prompt_token_ids)
        return (n + self.block_size - 1) // self.block_size * self.block_size - num_computed_tokens, True

    def update_state_after_alloc(self, req, num_external_tokens: int) -> None:
        p = req.kv_transfer_params or {}
        n_blocks = (len(req.prompt_token_ids) + self.block_size - 1) // self.block_size
        self._pending.append(ReqMeta(req.request_id, list(req.block_ids[:n_blocks]), list(p["remote_block_ids"][:n_blocks]),
                                     p["remote_host"], p.get("remote_engine_id", ""),
                                     window_block_ids=list(getattr(req, "omni_block_ids", None) or []),
                                     prompt_len=len(req.prompt_token_ids)))
        p["do_remote_prefill"] = False        # handled: a fallback re-schedule prefills locally

    def build_connector_meta(self) -> ConnectorMetadata:
        meta = ConnectorMetadata(self._pending)
        self._pending = []
        return meta

    def abandon(self, request_id: str) -> bool:
        """The scheduler wants to drop a request whose KV is being loaded.  Returns True when a transfer may be writing
        into its blocks: they must then stay allocated until the request shows up as received or failed."""
        before = len(self._pending)
        self._pending = [r for r in self._pending if r.request_id != request_id]
        if len(self._pending) != before:
            return False                      # never sent to the worker side: nothing is on its way
        return self.worker.abandon(request_id) if self.worker is not None else False

    def kick(self, meta: ConnectorMetadata) -> None:
        """Fast path: hand the metadata to the worker connector right away instead of with the next step."""
        if self.worker is not None and meta.requests:
            self.worker.bind_connector_metadata(meta)
            self.worker.start_load_kv()

    # -- producer
    def request_finished(self, req, block_ids: list):
        """Returns (delay_free, kv_transfer_params).  On a producer every request that ends at its token cap hands its
        KV over (the proxy's prefill leg is a plain request with max_tokens = 1 and no flag of its own, as in the
        reference's connector, llmdatadist_connector_v1.py:209-228); ``do_remote_decode: false`` opts a request out."""
        from ...engine.request import RequestStatus
        p = req.kv_transfer_params or {}
        if not (self.is_producer and p.get("do_remote_decode", True) and req.status == RequestStatus.FINISHED_LENGTH_CAPPED):
            return False, None
        n_blocks = (len(req.prompt_token_ids) + self.block_size - 1) // self.block_size
        params = {"do_remote_prefill": True, "do_remote_decode": False, "remote_block_ids": list(block_ids[:n_blocks]),
                  "remote_engine_id": self.engine_id, "remote_cluster_id": self.engine_id, "remote_host": self.endpoint,
                  "remote_host_ip": self.endpoint, "spec_token_ids": list(req.spec_token_ids) or [0] * self.num_spec,
                  "prompt_token_ids": list(req.prompt_token_ids),
                  "prefilled_token": req.output_token_ids[0] if req.output_token_ids else None}
        if self.worker is not None:
            self.worker.expect_pull(req.request_id)
        return True, params


# ------------------------------------------------------------------------------------------------ worker side
class WorkerConnector:
    SERVED_LIMIT = 4096          # producer: how many served request ids are remembered for re-acknowledgement

    def __init__(self, kv_role: str, engine_id: str, endpoint: str, transport: str = "inproc", sync_timeout_s: float = 20.0,
                 retries: int = 3, retry_wait_s: float = 2.0, authkey=None, handover_ttl_s: float = 120.0,
                 known_producers=None, known_consumers=None):
        self.kv_role, self.engine_id, self.endpoint, self.transport = kv_role, engine_id, endpoint, transport
        self.sync_timeout_s, self.retries, self.retry_wait_s = sync_timeout_s, retries, retry_wait_s
        self.handover_ttl_s = handover_ttl_s
        # with a deployment table (accelerators/pd/topology.py) KV is only asked from, and pushed to, instances it lists
        self.known_producers = set(known_producers) if known_producers else None
        self.known_consumers = set(known_consumers) if known_consumers else None
        self.refused_strangers = 0
        self.expired_handovers = 0         # producer: handed-over requests nobody asked for in time
        self.kv_tensors: list = []
        self._meta: Optional[ConnectorMetadata] = None
        self._lock = threading.Lock()
        self._done_recv: set = set()
        self._failed_recv: set = set()
        self._done_send: set = set()
        self._inflight: dict = {}          # consumer: request id -> (ReqMeta, attempt id)
        self._cancel_acked: set = set()    # consumer: (request id, attempt) whose cancel the producer confirmed
        self._abandoned: set = set()       # consumer: requests the scheduler dropped while their transfer was running
        self._attempts = 0
        self._expected: dict = {}          # producer: requests whose blocks wait to be pushed -> time of the hand-over
        self._served: dict = {}            # producer: request id -> attempt id of the push that was served (bounded)
        self._cancelled: set = set()       # producer: (request id, attempt) the consumer gave up on
        self._copying: set = set()         # producer: request ids whose copy is running right now
        self._peer_views: dict = {}        # producer: consumer endpoint -> cache view
        self.compressed_idx: list = []     # consumer with Omni-Attention: flat indices of the window-cache tensors
        self.omni_spec = None              # consumer with Omni-Attention: sink / recent / block size of a window
        self._tcp = None
        if transport == "inproc":
            InProcessHub.register(endpoint, self)
        else:
            self._tcp = TcpTransport(endpoint, self, authkey)

    # -- set-up
    def register_kv_caches(self, kv_caches, compressed_layers=None) -> None:
        """``compressed_layers``: indices (into ``kv_caches``) of the layers whose cache is a pool of per-request
        windows (Omni-Attention on a decode instance) rather than the paged cache."""
        self.kv_tensors = flatten_cache(kv_caches)
        comp, flat = set(compressed_layers or ()), 0
        self.compressed_idx = []
        for li, c in enumerate(kv_caches):
            n = len(c) if isinstance(c, (tuple, list)) else 1
            if li in comp:
                self.compressed_idx += list(range(flat, flat + n))
            flat += n

    def cache_descriptor(self) -> dict:
        """What a producer needs to write into this cache from another process (CUDA IPC handles)."""
        t0 = self.kv_tensors[0]
        desc = {"block_bytes": t0[0].numel() * t0.element_size(), "num_blocks": t0.shape[0], "n_tensors": len(self.kv_tensors),
                "num_blocks_per_tensor": [int(t.shape[0]) for t in self.kv_tensors]}
        if t0.is_cuda:
            from ...parallel.symmetric_heap import export_ipc_handles
            desc["ipc"] = export_ipc_handles(self.kv_tensors)
        return desc

    # -- step hooks used by the model runner
    def bind_connector_metadata(self, meta) -> None:
        self._meta = meta

    def start_load_kv(self) -> None:
        meta, self._meta = self._meta, None
        if meta is None:
            return
        for r in meta.requests:
            with self._lock:
                self._attempts += 1
                attempt = f"{self.engine_id}:{self._attempts}"
                self._inflight[r.request_id] = (r, attempt)
            threading.Thread(target=self._request_push, args=(r, attempt), daemon=True).start()

    def wait_for_save(self) -> None:
        """Producer side: blocks are written by the forward pass itself; nothing to flush."""

    def get_finished(self, finished_req_ids=None):
        with self._lock:
            if self._expected and self.handover_ttl_s > 0:
                limit = time.monotonic() - self.handover_ttl_s
                for rid in [k for k, t in self._expected.items() if t < limit and k not in self._copying]:
                    del self._expected[rid]
                    self._done_send.add(rid)
                    self.expired_handovers += 1
                    logger.warning("nobody asked for the KV of %s within %.0f s: blocks released", rid, self.handover_ttl_s)
            s, r = self._done_send, self._done_recv
            self._done_send, self._done_recv = set(), set()
        return s, r

    def take_failed(self) -> set:
        with self._lock:
            f, self._failed_recv = self._failed_recv, set()
        return f

    def abandon(self, request_id: str) -> bool:
        """Consumer: stop waiting for this request's KV.  True = a transfer is in flight; it is cancelled with the
        producer and the request is reported as failed (or received, if the copy won the race) once nothing can write
        into its blocks any more."""
        with self._lock:
            if self._meta is not None:
                n = len(self._meta.requests)
                self._meta.requests = [r for r in self._meta.requests if r.request_id != request_id]
                if len(self._meta.requests) != n:
                    return False              # bound but not started
            if request_id in self._inflight:
                self._abandoned.add(request_id)
                return True
        return False

    def expect_pull(self, request_id: str) -> None:
        with self._lock:
            self._expected[request_id] = time.monotonic()

    # -- message plumbing
    def dispatch(self, msg: dict) -> None:
        op = msg.get("op")
        if op == "push":
            self.handle_push_request(msg)
        elif op == "ack":
            self.handle_ack(msg)
        elif op == "nack":
            self.handle_nack(msg)
        elif op == "cancel":
            self.handle_cancel(msg)
        elif op == "cancel_ack":
            with self._lock:
                self._cancel_acked.add((msg["request_id"], msg.get("attempt")))
                if len(self._cancel_acked) > self.SERVED_LIMIT:      # confirmations that came after their wait had ended
                    self._cancel_acked.pop()

    def _send(self, endpoint: str, msg: dict) -> bool:
        if self.transport == "inproc":
            if msg["op"] == "push":
                return InProcessHub.send_push_request(endpoint, msg)
            if msg["op"] == "cancel":
                return InProcessHub.send_cancel(endpoint, msg)
            InProcessHub.send_ack(endpoint, msg)
            return True
        return self._tcp.send(endpoint, msg)

    # -- consumer: ask the producer to push, wait for the acknowledgement
    def _still_waiting(self, rid: str, attempt: str) -> bool:
        with self._lock:
            cur = self._inflight.get(rid)
            return cur is not None and cur[1] == attempt

    def _request_push(self, r: ReqMeta, attempt: str) -> None:
        msg = {"op": "push", "request_id": r.request_id, "attempt": attempt, "src_blocks": r.remote_block_ids,
               "dst_blocks": r.local_block_ids, "reply_to": self.endpoint, "consumer": self.engine_id}
        if self.transport != "inproc":
            msg["cache"] = self.cache_descriptor()
        if self.omni_spec is not None and self.compressed_idx and r.window_block_ids:
            sp = self.omni_spec
            msg["omni"] = {"sink": sp.sink, "recent": sp.recent, "block_size": sp.block_size, "prompt_len": r.prompt_len,
                           "dst_window": list(r.window_block_ids), "compressed": list(self.compressed_idx)}
        if self.known_producers is not None and r.remote_host not in self.known_producers:
            # the hand-over names an endpoint that is not a prefill instance of this deployment: nothing is asked of it
            logger.warning("kv for %s offered by %s, which the deployment table does not list: prefilling locally",
                           r.request_id, r.remote_host)
            with self._lock:
                self.refused_strangers += 1
                if self._inflight.get(r.request_id, (None, None))[1] == attempt:
                    del self._inflight[r.request_id]
                    self._failed_recv.add(r.request_id)
            return
        deadline = time.monotonic() + self.sync_timeout_s
        for n in range(self.retries + 1):
            self._send(r.remote_host, msg)
            # the last send waits out the whole synchronisation timeout, earlier ones one retry interval
            wait_until = deadline if n == self.retries else min(deadline, time.monotonic() + self.retry_wait_s)
            dropped = False
            while time.monotonic() < wait_until:
                if not self._still_waiting(r.request_id, attempt):
                    with self._lock:
                        self._abandoned.discard(r.request_id)
                    return                       # acknowledged, or refused by the producer
                with self._lock:
                    dropped = r.request_id in self._abandoned
                if dropped:
                    break
                time.sleep(0.002)
            if dropped or time.monotonic() >= deadline:
                break
            logger.warning("kv push for %s not acknowledged, retry %d", r.request_id, n + 1)
        # Give up.  A push that is still on its way must not land in blocks that were handed to another request:
        # tell the producer, and release the blocks only when it has confirmed (it waits for a running copy) or
        # stays silent for another retry interval (then it is gone and cannot write either).
        self._send(r.remote_host, {"op": "cancel", "request_id": r.request_id, "attempt": attempt, "reply_to": self.endpoint})
        t_end = time.monotonic() + max(self.retry_wait_s, 0.05)
        while time.monotonic() < t_end:
            with self._lock:
                if (r.request_id, attempt) in self._cancel_acked:
                    self._cancel_acked.discard((r.request_id, attempt))
                    break
            if not self._still_waiting(r.request_id, attempt):
                return                           # the acknowledgement overtook the cancel: the blocks are good
            time.sleep(0.002)
        with self._lock:
            cur = self._inflight.get(r.request_id)
            if cur is not None and cur[1] == attempt:
                del self._inflight[r.request_id]
                self._failed_recv.add(r.request_id)
            was_dropped = r.request_id in self._abandoned
            self._abandoned.discard(r.request_id)
        if was_dropped:
            logger.info("kv push for %s cancelled: the request was dropped", r.request_id)
        else:
            logger.error("kv push for %s abandoned after %.1fs", r.request_id, self.sync_timeout_s)

    def handle_ack(self, msg: dict) -> None:
        """Only the acknowledgement of the attempt that is being waited for counts: duplicates, strangers and late
        acknowledgements of an abandoned attempt are ignored."""
        with self._lock:
            cur = self._inflight.get(msg["request_id"])
            if cur is not None and msg.get("attempt", cur[1]) == cur[1]:
                del self._inflight[msg["request_id"]]
                self._done_recv.add(msg["request_id"])

    def handle_nack(self, msg: dict) -> None:
        """The producer does not know the request (it restarted, or freed the blocks): nothing was written, so the
        request goes to the local-prefill fallback at once instead of decoding on an empty cache."""
        with self._lock:
            cur = self._inflight.get(msg["request_id"])
            if cur is not None and msg.get("attempt", cur[1]) == cur[1]:
                del self._inflight[msg["request_id"]]
                self._failed_recv.add(msg["request_id"])

    # -- producer: copy the blocks into the consumer's cache, then acknowledge
    def _peer_cache(self, msg: dict):
        if self.transport == "inproc":
            return InProcessHub.endpoints[msg["reply_to"]].kv_tensors
        key = msg["reply_to"]
        if key not in self._peer_views:
            d = msg.get("cache") or {}
            if "ipc" not in d:
                # host tensors of another process cannot be mapped: refuse, so that the consumer prefills locally at once
                raise LookupError("the consumer's cache is not shareable between processes (no device IPC handles)")
            from ...parallel.symmetric_heap import open_ipc_handles
            self._peer_views[key] = PeerCacheView(open_ipc_handles(d["ipc"]), d["block_bytes"], d["num_blocks"])
            self._peer_views[key].num_blocks_per_tensor = d.get("num_blocks_per_tensor")
        return self._peer_views[key]

    def handle_push_request(self, msg: dict) -> None:
        rid, attempt = msg["request_id"], msg.get("attempt")
        if self.known_consumers is not None and msg.get("reply_to") not in self.known_consumers:
            logger.warning("push request for %s from %s, which the deployment table does not list: refused", rid, msg.get("reply_to"))
            with self._lock:
                self.refused_strangers += 1
            self._send(msg["reply_to"], {"op": "nack", "request_id": rid, "attempt": attempt})
            return
        with self._lock:
            if (rid, attempt) in self._cancelled:
                return                           # the consumer already gave this attempt up
            if rid in self._copying:
                return                           # a retry while the first copy is still running: one ack will follow
            served = self._served.get(rid, False)
            known = rid in self._expected
            if known:
                self._copying.add(rid)
        if not known:
            if served is not False and served == attempt:
                # a retry of the attempt that was served (its acknowledgement was lost): acknowledge again
                self._send(msg["reply_to"], {"op": "ack", "request_id": rid, "attempt": attempt})
            else:
                logger.warning("push request for unknown request %s refused", rid)
                self._send(msg["reply_to"], {"op": "nack", "request_id": rid, "attempt": attempt})
            return
        try:
            try:
                if msg.get("omni") and self.compressed_idx:
                    raise LookupError("a prefill instance with Omni-Attention has no full cache to send from")
                peer = self._peer_cache(msg)
            except LookupError as e:
                logger.warning("push request for %s refused: %s", rid, e)
                with self._lock:                 # the consumer prefills it itself now: the blocks are of no use here
                    if self._expected.pop(rid, None) is not None:
                        self._done_send.add(rid)
                self._send(msg["reply_to"], {"op": "nack", "request_id": rid, "attempt": attempt})
                return
            if msg.get("omni"):
                self._push_omni(peer, msg)
            elif isinstance(peer, PeerCacheView):
                push_blocks_cuda(self.kv_tensors, peer, msg["src_blocks"], msg["dst_blocks"])
            else:
                push_blocks_torch(self.kv_tensors, peer, msg["src_blocks"], msg["dst_blocks"])
                if self.kv_tensors and self.kv_tensors[0].is_cuda:
                    torch.cuda.synchronize()
        finally:
            with self._lock:
                self._copying.discard(rid)
        with self._lock:
            self._expected.pop(rid, None)
            self._done_send.add(rid)
            self._served[rid] = attempt
            while len(self._served) > self.SERVED_LIMIT:
                self._served.pop(next(iter(self._served)))
        self._send(msg["reply_to"], {"op": "ack", "request_id": rid, "attempt": attempt})

    def _push_omni(self, peer, msg: dict) -> None:
        """Transfer to a decode instance that runs Omni-Attention (reference: OmniBiGroupDataDistManager.pull_kv,
        omni/accelerators/cache/pd.py:81-123).  Full layers get the request's blocks as usual.  Compressed layers get
        only what their window keeps - the first ``sink`` blocks' worth of tokens and the most recent ones - token by
        token at the window positions the decode instance computes for a prompt of this length, so that its first step
        finds the window exactly as its own prefill would have left it."""
        from ..cache.omni_attn import OmniAttnConfig, OmniAttnState
        om = msg["omni"]
        bs, n_prompt = int(om["block_size"]), int(om["prompt_len"])
        comp = [int(i) for i in om["compressed"]]
        full = [i for i in range(len(self.kv_tensors)) if i not in set(comp)]
        src_blocks, dst_blocks, window = msg["src_blocks"], msg["dst_blocks"], om["dst_window"]
        st = OmniAttnState(OmniAttnConfig(int(om["sink"]), int(om["recent"]), 0.0, [1]), bs)
        src_slots, dst_slots = [], []
        for p in range(min(n_prompt, len(src_blocks) * bs)):
            w = st.window_position(p, n_prompt)
            if w is not None:
                src_slots.append(src_blocks[p // bs] * bs + p % bs)
                dst_slots.append(window[w // bs] * bs + w % bs)
        if isinstance(peer, PeerCacheView):
            per = getattr(peer, "num_blocks_per_tensor", None) or [peer.num_blocks] * len(peer.ptrs)
            if full:
                push_blocks_cuda([self.kv_tensors[i] for i in full],
                                 PeerCacheView([peer.ptrs[i] for i in full], peer.block_bytes, per[full[0]]), src_blocks, dst_blocks)
            if comp and src_slots:
                # the same copy kernel with one token as the unit: the caches seen as [slots, token bytes]
                toks = [self.kv_tensors[i].view(-1, *self.kv_tensors[i].shape[2:]) for i in comp]
                push_blocks_cuda(toks, PeerCacheView([peer.ptrs[i] for i in comp], peer.block_bytes // bs, per[comp[0]] * bs),
                                 src_slots, dst_slots)
            return
        if full:
            push_blocks_torch([self.kv_tensors[i] for i in full], [peer[i] for i in full], src_blocks, dst_blocks)
        if comp and src_slots:
            push_blocks_torch([self.kv_tensors[i].view(-1, *self.kv_tensors[i].shape[2:]) for i in comp],
                              [peer[i].view(-1, *peer[i].shape[2:]) for i in comp], src_slots, dst_slots)
        if self.kv_tensors and self.kv_tensors[0].is_cuda:
            torch.cuda.synchronize()

    def handle_cancel(self, msg: dict) -> None:
        rid, attempt = msg["request_id"], msg.get("attempt")
        with self._lock:
            self._cancelled.add((rid, attempt))
            if len(self._cancelled) > self.SERVED_LIMIT:
                self._cancelled.pop()
        # a copy of this request that is running right now finishes first: after the confirmation nothing of this
        # attempt is written any more
        t_end = time.monotonic() + 5.0
        while time.monotonic() < t_end:
            with self._lock:
                if rid not in self._copying:
                    break
            time.sleep(0.001)
        with self._lock:
            # the consumer gave the transfer up and prefills the request itself: nobody will ask for these blocks again
            if rid not in self._copying and self._expected.pop(rid, None) is not None:
                self._done_send.add(rid)
        self._send(msg["reply_to"], {"op": "cancel_ack", "request_id": rid, "attempt": attempt})

    def close(self) -> None:
        if self._tcp is not None:
            self._tcp.close()


def dump_thread_to_file(path: str) -> None:
    """Stack of every thread (connector threads included) for post-mortems."""
    import faulthandler
    with open(path, "w") as f:
        faulthandler.dump_traceback(file=f, all_threads=True)
