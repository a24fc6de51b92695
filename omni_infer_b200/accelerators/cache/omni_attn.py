"""Omni-Attention: KV-cache compression for decode (reference: omni/accelerators/cache/*.py).

A per-layer pattern marks layers as *compressed*: such a layer keeps, per request, only ``sink`` blocks from the
start of the sequence and a ring of ``recent`` blocks (defaults 1 and 3 blocks of 128 tokens,
kv_cache_interface.py:27-30).  Its KV memory is constant in the sequence length.  Full layers use the ordinary
paged cache.  Two block pools exist (kv_cache_manager.py:62-484): the ordinary one, and one from which every
request takes exactly ``sink + recent`` blocks once, for all compressed layers.  Prefix caching is off.

Slot of a token in a compressed layer (cache/utils.py:36-50): while the sequence fits (length <= (sink+recent)
blocks) positions are linear; afterwards the token wraps inside the recent window,
``window_pos = (L - base) % recent_tokens + sink_tokens`` with ``base = max(capacity, prompt_len) + 1``.
A prompt longer than the capacity stores its first ``sink_tokens`` tokens and its last ``recent_tokens`` tokens, so
that the first generated token overwrites the oldest window entry.  Attention in a compressed layer runs over
``min(L, capacity)`` tokens through the request's small block table; the order of keys inside the window does not
matter because RoPE was applied with the true positions when they were written."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ... import ops
from ...engine.kv_manager import KVCacheManager

SINK, RECENT, BETA = 1, 3, 0.2


def default_pattern(num_layers: int, beta: float = BETA) -> list:
    """Every layer compressed except the first ones and a share ``beta`` spread evenly (the reference ships a
    fixed 61-entry list; this reproduces its density for any depth)."""
    keep_every = max(1, int(round(1.0 / max(beta, 1e-6))))
    return [0 if (i < 2 or i % keep_every == 0) else 1 for i in range(num_layers)]


@dataclass
class OmniAttnConfig:
    sink: int = SINK
    recent: int = RECENT
    beta: float = BETA
    pattern: Optional[list] = None

    @classmethod
    def from_dict(cls, d: Optional[dict], num_layers: int) -> "OmniAttnConfig":
        d = d or {}
        c = cls(int(d.get("sink", SINK)), int(d.get("recent", RECENT)), float(d.get("beta", BETA)), d.get("pattern"))
        if c.pattern is None:
            c.pattern = default_pattern(num_layers, c.beta)
        if len(c.pattern) != num_layers:
            raise ValueError(f"omni_attn pattern has {len(c.pattern)} entries for {num_layers} layers")
        return c


@dataclass
class OmniAttentionSpec:
    """KV spec of a compressed layer: fixed number of blocks per request."""
    block_size: int
    sink: int
    recent: int

    @property
    def blocks_per_request(self) -> int:
        return self.sink + self.recent

    @property
    def capacity_tokens(self) -> int:
        return self.blocks_per_request * self.block_size


class OmniKVCacheManager(KVCacheManager):
    """Two pools: the ordinary paged pool (full layers) and a pool of fixed-size per-request windows (compressed
    layers).  ``req.omni_block_ids`` holds the window of a request."""

    def __init__(self, num_blocks: int, block_size: int, spec: OmniAttentionSpec, num_window_blocks: int):
        super().__init__(num_blocks, block_size, enable_prefix_caching=False)
        self.spec = spec
        self.window_free = list(range(1, num_window_blocks))      # block 0 = padding target
        self.num_window_blocks = num_window_blocks

    def allocate_slots(self, req, num_new_tokens, computed_blocks=None, lookahead=0):
        need_window = not getattr(req, "omni_block_ids", None)
        if need_window and len(self.window_free) < self.spec.blocks_per_request:
            return None
        new = super().allocate_slots(req, num_new_tokens, computed_blocks, lookahead)
        if new is None:
            return None
        if need_window:
            n = self.spec.blocks_per_request
            req.omni_block_ids, self.window_free = self.window_free[:n], self.window_free[n:]
        return new

    def free(self, req) -> None:
        super().free(req)
        w = getattr(req, "omni_block_ids", None)
        if w:
            self.window_free.extend(w)
            req.omni_block_ids = []


class OmniAttnState:
    """Runner-side helper: which layers are compressed and how to build their slot mapping / block tables."""

    def __init__(self, cfg: OmniAttnConfig, block_size: int):
        self.cfg, self.block_size = cfg, block_size
        self.spec = OmniAttentionSpec(block_size, cfg.sink, cfg.recent)
        self.pattern = list(cfg.pattern)

    def is_compressed(self, layer_idx: int) -> bool:
        return layer_idx < len(self.pattern) and bool(self.pattern[layer_idx])

    # ---- prefill: where each token goes in the window (or -1)
    def window_position(self, p: int, prompt_len: int):
        """Window position that the token at sequence position ``p`` is written to, or None for a prompt token that is
        not kept.  Prompt tokens follow the prefill rule, generated ones the decode ring."""
        st, rt = self.cfg.sink * self.block_size, self.cfg.recent * self.block_size
        cap = st + rt
        if p >= prompt_len:
            return compute_omni_attn_metadata_ref(p + 1, prompt_len, self.block_size, self.cfg.sink, self.cfg.recent)[0]
        if prompt_len <= cap or p < st:
            return p
        if p >= prompt_len - rt:
            return st + (p - (prompt_len - rt))
        return None

    def prefill_slots(self, window_blocks: list, start: int, n: int, prompt_len: int, total_len: Optional[int] = None) -> list:
        """Slots of the tokens ``[start, start + n)`` of a prefill over ``total_len`` tokens (default: the prompt).  A
        request that was preempted recomputes its prompt *and* what it had generated (``total_len > prompt_len``); the
        generated tokens then go where the decode steps had put them, and a token whose window entry a later one of the
        same prefill takes is not written at all (the scatter has no order), so that the window ends up as the decode
        steps had left it."""
        bs = self.block_size
        total = prompt_len if total_len is None else max(total_len, prompt_len)
        last_writer = {}
        if total > prompt_len:
            for p in range(total):
                w = self.window_position(p, prompt_len)
                if w is not None:
                    last_writer[w] = p
        out = []
        for p in range(start, start + n):
            w = self.window_position(p, prompt_len)
            if w is None or (last_writer and last_writer.get(w) != p):
                out.append(-1)
                continue
            out.append(window_blocks[w // bs] * bs + w % bs)
        return out

    # ---- decode: slot of the new token and attended length, on device
    def decode_metadata(self, seq_lens: torch.Tensor, prompt_lens: torch.Tensor, window_table: torch.Tensor):
        slots, eff = ops.omni_attn_slots(seq_lens, prompt_lens, window_table, self.block_size, self.cfg.sink, self.cfg.recent)
        return {"slot_mapping": slots, "q_seq_lens": eff, "block_table": window_table,
                "max_seq_len": self.spec.capacity_tokens}

    # ---- PD: which blocks of a finished prefill must travel for compressed layers (cache/pd.py:81-123)
    def select_transfer_blocks(self, src_blocks: list, prompt_len: int, dst_window: list) -> list:
        """Pairs (src_block, dst_window_block): the sink blocks and the last ``recent`` prompt blocks."""
        nb = (prompt_len + self.block_size - 1) // self.block_size
        pairs = [(src_blocks[i], dst_window[i]) for i in range(min(self.cfg.sink, nb))]
        tail = list(range(max(self.cfg.sink, nb - self.cfg.recent), nb))
        for j, i in enumerate(tail):
            pairs.append((src_blocks[i], dst_window[self.cfg.sink + j]))
        return pairs


def compute_omni_attn_metadata_ref(seq_len: int, prompt_len: int, block_size: int, sink: int = SINK, recent: int = RECENT):
    """Scalar reference of the ring-window position (tests)."""
    st, rt = sink * block_size, recent * block_size
    cap = st + rt
    if seq_len <= cap:
        return seq_len - 1, seq_len
    base = max(cap, prompt_len) + 1
    return (seq_len - base) % rt + st, cap
