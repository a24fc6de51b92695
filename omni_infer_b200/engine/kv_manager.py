"""Paged KV-cache block manager: free list, reference counts, optional hash-based prefix caching.

Block size defaults to 128 tokens as in the reference deployment (omni/adaptors/vllm/platform.py:226).
Block 0 is reserved as the padding target of CUDA-graph padded rows."""
from __future__ import annotations

import hashlib
from collections import OrderedDict, deque
from typing import Optional

from .request import Request


class KVCacheManager:
    def __init__(self, num_blocks: int, block_size: int = 128, enable_prefix_caching: bool = False,
                 reserve_null_block: bool = True):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.enable_prefix_caching = enable_prefix_caching
        first = 1 if reserve_null_block else 0
        self.free_blocks: deque = deque(range(first, num_blocks))
        self.ref: list = [0] * num_blocks
        self.hash_to_block: dict = {}
        self.block_hash: dict = {}
        self.evictable: OrderedDict = OrderedDict()    # cached, unreferenced blocks in LRU order

    # ------------------------------------------------------------------ accounting
    @property
    def num_free_blocks(self) -> int:
        return len(self.free_blocks) + len(self.evictable)

    @property
    def usage(self) -> float:
        total = self.num_blocks - 1
        return 1.0 - self.num_free_blocks / max(total, 1)

    def blocks_needed(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def _pop_free(self) -> Optional[int]:
        if self.free_blocks:
            return self.free_blocks.popleft()
        if self.evictable:
            b, _ = self.evictable.popitem(last=False)
            h = self.block_hash.pop(b, None)
            if h is not None and self.hash_to_block.get(h) == b:
                del self.hash_to_block[h]
            return b
        return None

    # ------------------------------------------------------------------ prefix cache
    def _hash_chain(self, token_ids: list):
        prev = b""
        for i in range(0, len(token_ids) - len(token_ids) % self.block_size, self.block_size):
            m = hashlib.sha256(prev)
            m.update(str(token_ids[i:i + self.block_size]).encode())
            prev = m.digest()
            yield prev

    def get_computed_blocks(self, req: Request) -> tuple:
        """Longest cached prefix (full blocks only, never the whole prompt: the last token must run)."""
        if not self.enable_prefix_caching:
            return [], 0
        blocks = []
        for h in self._hash_chain(req.prompt_token_ids[:-1]):
            b = self.hash_to_block.get(h)
            if b is None:
                break
            blocks.append(b)
        return blocks, len(blocks) * self.block_size

    def cache_full_blocks(self, req: Request) -> None:
        if not self.enable_prefix_caching:
            return
        n_full = req.num_computed_tokens // self.block_size
        for i, h in enumerate(self._hash_chain(req.all_token_ids[: n_full * self.block_size])):
            b = req.block_ids[i]
            if b not in self.block_hash and h not in self.hash_to_block:
                self.block_hash[b] = h
                self.hash_to_block[h] = b

    # ------------------------------------------------------------------ allocation
    def allocate_slots(self, req: Request, num_new_tokens: int, computed_blocks: Optional[list] = None,
                       lookahead: int = 0) -> Optional[list]:
        """Make sure ``req`` owns blocks for ``num_computed_tokens + num_new_tokens + lookahead`` tokens.
        Returns the newly added block ids, or None when memory is short (nothing is changed then)."""
        took_prefix = bool(computed_blocks) and not req.block_ids
        if took_prefix:
            for b in computed_blocks:
                self.ref[b] += 1
                self.evictable.pop(b, None)
            req.block_ids = list(computed_blocks)
        need = self.blocks_needed(req.num_computed_tokens + num_new_tokens + lookahead) - len(req.block_ids)
        if need <= 0:
            return []
        if need > self.num_free_blocks:
            if took_prefix:
                self.free(req)      # give the cached-prefix references back: a failed call leaves no trace
            return None
        new = []
        for _ in range(need):
            b = self._pop_free()
            self.ref[b] = 1
            new.append(b)
        req.block_ids.extend(new)
        return new

    def free(self, req: Request) -> None:
        for b in reversed(req.block_ids):
            if self.ref[b] <= 0:
                continue      # tolerated double free (a finished_sending ack may race a finish)
            self.ref[b] -= 1
            if self.ref[b] == 0:
                if b in self.block_hash:
                    self.evictable[b] = True
                else:
                    self.free_blocks.append(b)
        req.block_ids = []

    def get_block_ids(self, req: Optional[Request]) -> list:
        """Unknown requests answer with an empty group instead of raising (the KV connector may ask about a
        request the scheduler already dropped)."""
        return [list(req.block_ids)] if req is not None else [[]]
