"""OmniPlanner: facade over the placement core used by the MoE layers and the model runner
(reference: omni_planner/omni_planner.py:45-343, placement_handler.py:32-156).

* ``selector(layer)`` - int32 device row mapping logical to physical expert ids; the router kernel applies it
  (the reference does ``F.embedding(topk_ids, expert_mapping)`` in ``plan``).
* ``activation_counts(layer)`` - int64 device row incremented by the router kernel per physical position.
* ``place_experts(min_ready)`` - called by the runner before every step, right after the ranks' per-step agreement on
  the host group, which also carries the minimum over the ranks of ``ready_rounds()``: a re-placement round is applied
  (weights copied from staging, selector refreshed) in the step in which every rank has it complete, by all ranks at
  that same step boundary.
* ``init_dram_weights(model)`` - registers the expert tensors (w13 / w2 and their scales) of every local slot.
* ``start_dynamic_optimize_expert_load_balance()`` - starts the C++ background thread.

Configuration keys follow the reference's ``config.yaml``: ``pattern_path``, ``max_moe_layer_num``,
``enable_dynamic``, ``max_redundant_per_expert``, ``max_redundant_per_rank``, ``enable_dump``, ``dump_dir``."""
from __future__ import annotations

import ctypes
import logging
import os
import threading
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ...parallel import get_parallel_state
from . import _native as nat
from .expert_mapping import ExpertMapping

logger = logging.getLogger("omni_infer_b200.placement")


class _Singleton(type):
    _inst = None
    _lock = threading.Lock()

    def __call__(cls, *a, **kw):
        with cls._lock:
            fresh = kw.pop("_new", False)
            if cls._inst is None or fresh:
                cls._inst = super().__call__(*a, **kw)
        return cls._inst

    def cleanup(cls):
        with cls._lock:
            if cls._inst is not None:
                cls._inst.close()
            cls._inst = None


class OmniPlanner(metaclass=_Singleton):
    def __init__(self, num_moe_layers: int, num_experts: int, device="cpu", pattern: Optional[np.ndarray] = None,
                 max_redundant_per_rank: int = 0, max_redundant_per_expert: int = 10, enable_dynamic: bool = False,
                 period_s: float = 60.0, apply_interval: int = 16, enable_dump: bool = False, dump_dir: str = "",
                 ranks_per_host: int = 8, host_replica: str = ""):
        ps = get_parallel_state()
        self.world, self.rank = ps.ep_size, ps.ep_rank
        self.device = torch.device(device)
        self.layers, self.experts = num_moe_layers, num_experts
        self.num_redundant_per_rank = max_redundant_per_rank
        self.max_redundant_per_expert = max_redundant_per_expert
        self.enable_dynamic, self.period_s, self.apply_interval = enable_dynamic, period_s, apply_interval
        self.enable_dump, self.dump_dir = enable_dump, dump_dir
        # name of a POSIX shared-memory segment that holds every expert once per host (the reference's second
        # replacement variant): an expert is then replaced by a host -> device copy on the rank that wants it
        self.host_replica, self.ranks_per_host = host_replica, ranks_per_host
        self.mapping = ExpertMapping(pattern, self.world, self.rank, num_moe_layers, num_experts, max_redundant_per_rank,
                                     ranks_per_host, device)
        self.slots_per_rank = self.mapping.slots_per_rank
        self.num_positions = self.world * self.slots_per_rank
        # tokens this rank routed to every physical position (router kernel), and the cluster-wide totals of the
        # positions this rank owns (what the C++ ClusterActivation reads)
        self.sent_counts = torch.zeros(num_moe_layers, self.num_positions, dtype=torch.int64, device=self.device)
        self.local_counts = torch.zeros(num_moe_layers, self.slots_per_rank, dtype=torch.int64, device=self.device)
        self._step = 0
        self._applied_round = 0      # placement rounds applied so far (compared with ready_rounds of all ranks)
        self.applied_total = 0    # experts replaced since start (all rounds)
        self._weights = self._act = self._dist = self._placement = None
        self._keep = []          # ctypes callbacks must outlive the C++ objects
        self._pl_group = None
        self._install_copy_hooks()

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_config(cls, cfg: dict, model_cfg) -> "OmniPlanner":
        if "config_path" in cfg:
            import yaml
            cfg = dict(yaml.safe_load(open(cfg["config_path"])) or {}, **{k: v for k, v in cfg.items() if k != "config_path"})
        layers = model_cfg.num_hidden_layers - model_cfg.first_k_dense_replace
        layers = min(layers, int(cfg.get("max_moe_layer_num", layers)))
        pattern = cfg.get("pattern")          # an array handed over directly (restored state)
        if cfg.get("pattern_path"):
            pattern = np.load(cfg["pattern_path"])
        dev = "cuda" if torch.cuda.is_available() and os.environ.get("NO_GPU_MOCK", "0") != "1" else "cpu"
        return cls(layers, model_cfg.n_routed_experts, device=cfg.get("device", dev), pattern=pattern,
                   max_redundant_per_rank=int(cfg.get("max_redundant_per_rank", 0)),
                   max_redundant_per_expert=int(cfg.get("max_redundant_per_expert", 10)),
                   enable_dynamic=bool(cfg.get("enable_dynamic", False)), period_s=float(cfg.get("period_s", 60.0)),
                   apply_interval=int(cfg.get("apply_interval", 16)), enable_dump=bool(cfg.get("enable_dump", False)),
                   dump_dir=cfg.get("dump_dir", ""), ranks_per_host=int(cfg.get("ranks_per_host", 8)),
                   host_replica=str(cfg.get("host_replica", "")), _new=True)

    def _install_copy_hooks(self) -> None:
        L = nat.lib()
        if self.device.type != "cuda":
            L.omni_pl_set_ut_memcpy()
            return
        rt = ctypes.CDLL("libcudart.so.12")
        rt.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        rt.cudaStreamSynchronize.argtypes = [ctypes.c_void_p]
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._rt, self._dev_index = rt, dev_index
        # copies of the placement machinery run on their own low-priority, non-blocking stream: they never order
        # themselves against the inference streams, and a copy only blocks the thread that asked for it
        lo, _hi = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, "priority_range") else (0, -1)
        self._copy_stream = torch.cuda.Stream(device=self.device, priority=lo)
        stream_ptr = ctypes.c_void_p(self._copy_stream.cuda_stream)

        def mk(kind):
            def f(dst, src, n):
                rt.cudaSetDevice(dev_index)       # the background thread has no current device yet
                rc = rt.cudaMemcpyAsync(dst, src, n, kind, stream_ptr)
                rc = rc or rt.cudaStreamSynchronize(stream_ptr)
                if rc != 0:
                    logger.error("cudaMemcpyAsync(kind=%d) failed with %d", kind, rc)
            return nat.COPY_FN(f)

        hooks = (mk(3), mk(1), mk(2))      # d2d, h2d, d2h
        self._keep += list(hooks)
        L.omni_pl_set_copy_hooks(*hooks)

    # ------------------------------------------------------------------ per-layer accessors (hot path)
    def selector(self, moe_layer: int) -> torch.Tensor:
        return self.mapping.selector_dev[min(moe_layer, self.layers - 1)]

    def activation_counts(self, moe_layer: int) -> torch.Tensor:
        return self.sent_counts[min(moe_layer, self.layers - 1)]

    def plan(self, moe_layer: int, topk_ids: torch.Tensor) -> torch.Tensor:
        """Reference-compatible call: logical ids -> physical ids."""
        return torch.nn.functional.embedding(topk_ids.long(), self.selector(moe_layer).unsqueeze(-1)).squeeze(-1).int()

    def record_activation(self, moe_layer: int, expert_token_nums: torch.Tensor) -> None:
        """Add tokens received per local slot (used by paths that do not route through the fused router)."""
        base = self.rank * self.slots_per_rank
        self.sent_counts[moe_layer, base:base + self.slots_per_rank] += expert_token_nums.to(torch.int64)

    def local_slots_of(self, moe_layer: int, expert: int) -> list:
        return self.mapping.local_slots_of(min(moe_layer, self.layers - 1), expert)

    def logical_of_slot(self, moe_layer: int, slot: int) -> int:
        e = self.mapping.logical_of_slot(min(moe_layer, self.layers - 1), slot)
        return e if e >= 0 else self.experts + self.rank * self.slots_per_rank + slot   # empty slot: unique filler id

    def is_expert_on_current_rank(self, moe_layer: int, expert: int) -> bool:
        return self.mapping.is_expert_on_current_rank(min(moe_layer, self.layers - 1), expert)

    def get_num_of_redundant_experts(self, moe_layer: int = 0) -> int:
        return self.mapping.get_num_of_redundant_experts(moe_layer)

    # ------------------------------------------------------------------ weights / dynamic loop
    def init_dram_weights(self, model) -> None:
        """Register w13 / w2 (and scale) tensors of every local slot with the C++ registry."""
        L = nat.lib()
        self._weights = L.omni_pl_weights_create(self.layers, self.slots_per_rank)
        for mod in model.modules():
            if mod.__class__.__name__ != "MoELayer" or mod.moe_index >= self.layers:
                continue
            for name in ("w13", "w13_scale", "w2", "w2_scale"):
                t = getattr(mod, name, None)
                if t is None:
                    continue
                for s in range(self.slots_per_rank):
                    sl = t.data[s]
                    L.omni_pl_weights_add(self._weights, mod.moe_index, s, ctypes.c_void_p(sl.data_ptr()),
                                          sl.numel() * sl.element_size())
        L.omni_pl_weights_set_initialized(self._weights)
        if self.host_replica:
            on_host = min(self.ranks_per_host, self.world)
            if L.omni_pl_weights_init_shm(self._weights, self.host_replica.encode(), self.experts, on_host) != 0:
                raise RuntimeError(f"cannot create or attach the expert replica {self.host_replica!r}")
            L.omni_pl_weights_replicate(self._weights, self.mapping.handle)
            logger.info("expert replica %s: %.1f MiB of host memory", self.host_replica,
                        L.omni_pl_weights_replica_bytes(self._weights) / 2 ** 20)
        self._act = L.omni_pl_activation_create(ctypes.c_void_p(self.local_counts.data_ptr()), self.layers,
                                                self.slots_per_rank, self.world, self.rank, 8)
        if self.enable_dynamic:
            self.start_dynamic_optimize_expert_load_balance()

    def _make_distribution(self):
        L = nat.lib()
        eb = L.omni_pl_weights_expert_bytes(self._weights)
        world, rank = self.world, self.rank
        if world > 1 and self._pl_group is None:
            self._pl_group = dist.new_group(list(range(world)), backend="gloo")   # private: used from the C++ thread
        g = self._pl_group

        def allgather(send, recv, n):
            s = torch.frombuffer((ctypes.c_longlong * n).from_address(send), dtype=torch.int64)
            r = torch.frombuffer((ctypes.c_longlong * (n * world)).from_address(recv), dtype=torch.int64)
            if world == 1:
                r.copy_(s)
            else:
                dist.all_gather_into_tensor(r, s.clone(), group=g)

        def sendrecv(peer, send, recv, n):
            ops = []
            if send:
                sb = torch.frombuffer((ctypes.c_ubyte * n).from_address(send), dtype=torch.uint8)
                ops.append(dist.P2POp(dist.isend, sb, peer, g))
            if recv:
                rb = torch.frombuffer((ctypes.c_ubyte * n).from_address(recv), dtype=torch.uint8)
                ops.append(dist.P2POp(dist.irecv, rb, peer, g))
            # lower rank posts send first, higher rank receive first (pairwise ordering, as the reference's swap)
            if rank > peer:
                ops.reverse()
            for w in dist.batch_isend_irecv(ops):
                w.wait()

        def barrier():
            if world > 1:
                dist.barrier(group=g)

        if self.device.type == "cuda" and world > 1 and os.environ.get("OMNI_PLACEMENT_HOST_STAGING", "0") != "1":
            return self._make_device_distribution(eb, allgather, barrier)
        cbs = (nat.ALLGATHER_FN(allgather), nat.SENDRECV_FN(sendrecv), nat.BARRIER_FN(barrier))
        self._keep += list(cbs)
        return L.omni_pl_distribution_create(rank, world, eb, *cbs)

    def _make_device_distribution(self, expert_bytes: int, allgather, barrier):
        """Expert weights travel over the device fabric (reference: rank-ordered device Send/Recv into a ring of five
        staging buffers, omni/accelerators/placement/omni_planner/cpp/distribution.cpp:173-218, moe_weights.cpp:32-101).

        Every rank owns one send buffer (a packed expert, exported with CUDA IPC and mapped by all peers) and five
        staging buffers.  To move an expert the source packs it into its send buffer with device copies and tells the
        destination over the host group that it is ready; the destination pulls it across NVLink into a staging
        buffer with an asynchronous peer copy on the placement stream (copy engines, no SM kernel, nothing ordered
        against the inference streams) and acknowledges, so that the send buffer can be reused.  The inference
        thread later copies staging -> live weights on the device between two steps."""
        from ...parallel.symmetric_heap import alloc_ipc_tensor, export_ipc_handles, open_ipc_handles
        L = nat.lib()
        world, rank, g = self.world, self.rank, self._pl_group
        nbytes = (int(expert_bytes) + 255) // 256 * 256
        self._send_buf = alloc_ipc_tensor((nbytes,), torch.uint8)
        self._stages = [torch.empty(nbytes, dtype=torch.uint8, device=self.device) for _ in range(5)]
        handles = [None] * world
        dist.all_gather_object(handles, export_ipc_handles([self._send_buf])[0], group=g)
        self._peer_send = [open_ipc_handles([h])[0] if r != rank else self._send_buf.data_ptr() for r, h in enumerate(handles)]
        rt, stream_ptr = self._rt, ctypes.c_void_p(self._copy_stream.cuda_stream)
        tok = torch.zeros(1, dtype=torch.int64)

        def exchange(peer, sending, receiving):
            """One small host message each way that applies: 'my buffer is ready' / 'I am done with yours'."""
            ops = []
            if sending:
                ops.append(dist.P2POp(dist.isend, tok.clone(), peer, g))
            if receiving:
                ops.append(dist.P2POp(dist.irecv, torch.empty_like(tok), peer, g))
            if rank > peer:
                ops.reverse()
            for w in dist.batch_isend_irecv(ops):
                w.wait()

        def sendrecv(peer, send, recv, n):
            rt.cudaSetDevice(self._dev_index)
            has_send, has_recv = bool(send), bool(recv)
            exchange(peer, has_send, has_recv)             # data packed on the sender(s)
            if has_recv:
                rc = rt.cudaMemcpyAsync(recv, ctypes.c_void_p(self._peer_send[peer]), n, 3, stream_ptr)
                rc = rc or rt.cudaStreamSynchronize(stream_ptr)
                if rc != 0:
                    logger.error("peer copy of an expert from rank %d failed with %d", peer, rc)
            exchange(peer, has_recv, has_send)             # readers are done: send buffers may be reused

        cbs = (nat.ALLGATHER_FN(allgather), nat.SENDRECV_FN(sendrecv), nat.BARRIER_FN(barrier))
        self._keep += list(cbs)
        stage_ptrs = (ctypes.c_void_p * 5)(*[ctypes.c_void_p(t.data_ptr()) for t in self._stages])
        self._keep.append(stage_ptrs)
        return L.omni_pl_distribution_create_device(rank, world, expert_bytes, *cbs, ctypes.c_void_p(self._send_buf.data_ptr()),
                                                    stage_ptrs)

    def _ensure_placement(self):
        if self._placement is None:
            L = nat.lib()
            self._dist = self._make_distribution()
            self._placement = L.omni_pl_placement_create(self.mapping.handle, self._weights, self._act, self._dist,
                                                         self.max_redundant_per_expert, self.period_s)
            self._restore_ema()
        return self._placement

    # ------------------------------------------------------------------ state kept across restarts
    pending_ema = None         # (saved positions [layers, P], saved averages [layers, P]) or a bare average array

    def export_state(self) -> dict:
        """What a restart needs to continue where this run stands: the placement as a 0/1 pattern (the start-up
        format), the same placement position by position, and the balancer's moving average of position loads."""
        from .expert_mapping import pattern_from_placement
        placement = self.mapping.placement()
        out = {"placement_pattern": pattern_from_placement(placement, self.world, self.slots_per_rank, self.experts),
               "placement_positions": placement}
        if self._placement is not None:
            buf = np.zeros(self.layers * self.num_positions, dtype=np.float64)
            n = nat.lib().omni_pl_placement_get_ema(self._placement, buf.ctypes.data, buf.size)
            if n == buf.size:
                out["placement_ema"] = buf.reshape(self.layers, self.num_positions)
        return out

    def _restore_ema(self) -> None:
        """Hands a saved moving average to the new balancer.  A placement restored from its pattern fills each rank's
        slots in expert order, which need not be the order they had when the average was saved, so the values are
        carried over by (layer, rank, expert), not by position."""
        pend = self.pending_ema
        self.pending_ema = None
        if pend is None:
            return
        saved_pos, ema = pend if isinstance(pend, tuple) else (None, pend)
        ema = np.asarray(ema, dtype=np.float64)
        if ema.shape != (self.layers, self.num_positions):
            logger.info("saved load history has shape %s, this deployment needs %s: ignored", ema.shape,
                        (self.layers, self.num_positions))
            return
        now = self.mapping.placement()
        if saved_pos is not None and np.asarray(saved_pos).shape == now.shape and not np.array_equal(saved_pos, now):
            S, remapped = self.slots_per_rank, np.zeros_like(ema)
            for l in range(self.layers):
                for r in range(self.world):
                    old = {int(e): ema[l, r * S + k] for k, e in enumerate(saved_pos[l, r * S:(r + 1) * S]) if e >= 0}
                    for k, e in enumerate(now[l, r * S:(r + 1) * S]):
                        remapped[l, r * S + k] = old.get(int(e), 0.0)
            ema = remapped
        ema = np.ascontiguousarray(ema)
        if nat.lib().omni_pl_placement_set_ema(self._placement, ema.ctypes.data, ema.size) != 0:
            logger.warning("the balancer refused the saved load history")

    def start_dynamic_optimize_expert_load_balance(self) -> None:
        nat.lib().omni_pl_placement_start(self._ensure_placement())

    def sync_activation_counts(self) -> None:
        """Cluster-wide totals of this rank's positions -> ``local_counts`` (read by the C++ collector)."""
        tot = self.sent_counts.clone()
        if self.world > 1:
            dist.all_reduce(tot, group=get_parallel_state().group("world").group)
        base = self.rank * self.slots_per_rank
        self.local_counts.copy_(tot[:, base:base + self.slots_per_rank] % (10 ** 16))

    def run_round(self) -> int:
        """One synchronous optimisation round (tests, offline use)."""
        self.sync_activation_counts()
        return nat.lib().omni_pl_placement_run_round(self._ensure_placement())

    def ready_rounds(self) -> int:
        """Placement rounds that are complete on this rank (staged on every rank, published after the round's barrier)."""
        return int(nat.lib().omni_pl_placement_ready_rounds(self._placement)) if self._placement else 0

    def place_experts(self, min_ready: Optional[int] = None) -> int:
        """Between steps: keep the collector's input fresh and apply a finished round.  ``min_ready`` = the smallest
        ``ready_rounds()`` of any rank, exchanged by the caller: a round is applied when every rank has it complete, by
        all of them in the same step.  Without it (one rank, or a caller that steps all ranks itself) the rank goes by
        its own counter."""
        self._step += 1
        if self._placement is None:
            return 0
        if self._step % self.apply_interval == 0:
            self.sync_activation_counts()
        ready = self.ready_rounds() if min_ready is None else int(min_ready)
        if ready <= self._applied_round:
            return 0
        self._applied_round = ready
        return self.apply_pending()

    def apply_pending(self) -> int:
        L = nat.lib()
        n = L.omni_pl_do_placement_optimizer(self._placement)
        self.applied_total += int(n)
        self.mapping.refresh_selector()
        if self.enable_dump and self.dump_dir:
            os.makedirs(self.dump_dir, exist_ok=True)
            L.omni_pl_activation_dump(self._act, os.path.join(self.dump_dir, f"activation_rank{self.rank}_{self._step}.txt").encode())
        return n

    def last_instructions(self) -> list:
        buf = (ctypes.c_int * (8 * 256))()
        n = nat.lib().omni_pl_placement_last_instructions(self._placement, buf, 256)
        names = ("layer", "type", "source_rank", "source_expert", "source_pos", "target_rank", "target_expert", "target_pos")
        return [dict(zip(names, buf[8 * i:8 * i + 8])) for i in range(n)]

    def load_stats(self, since: Optional[torch.Tensor] = None) -> dict:
        """max / mean tokens per rank and per expert position over the accumulated counters (placement gauges);
        ``since`` = an earlier copy of ``sent_counts`` restricts the gauges to what was counted after it."""
        c = (self.sent_counts if since is None else self.sent_counts - since).float()
        if self.world > 1 and dist.is_initialized():
            c = c.clone()
            dist.all_reduce(c, group=get_parallel_state().group("world").group)
        per_rank = c.view(self.layers, self.world, self.slots_per_rank).sum(-1)
        return {"max_over_mean_rank_load": float((per_rank.max(-1).values / per_rank.mean(-1).clamp_min(1e-9)).mean()),
                "max_over_mean_position_load": float((c.max(-1).values / c.mean(-1).clamp_min(1e-9)).mean())}

    def close(self) -> None:
        L = nat.lib()
        if self._placement:
            L.omni_pl_placement_stop(self._placement)
            L.omni_pl_placement_destroy(self._placement)
            self._placement = None
        if self._dist:
            L.omni_pl_distribution_destroy(self._dist)
            self._dist = None
        if self._act:
            L.omni_pl_activation_destroy(self._act)
            self._act = None
        if self._weights:
            if self.host_replica:
                L.omni_pl_weights_close_shm(self._weights, 1 if self.rank % max(self.ranks_per_host, 1) == 0 else 0)
            L.omni_pl_weights_destroy(self._weights)
            self._weights = None
        self.mapping.close()
