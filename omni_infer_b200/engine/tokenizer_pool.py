"""Tokenisation front end.  Long prompts are tokenised in a pool of worker processes pinned to chosen CPU cores so
that the API server's event loop is not blocked (reference: tokenizer_proc_pool.patch; env TOKENIZER_PROC_POOL,
TOKENIZER_WORKER_NUM, TOKENIZER_PROC_POOL_THRES, TOKENIZER_AFFINITY_CORES).  Without a tokenizer directory a
byte-level fallback is used (token = byte value mod vocab), which keeps the serving stack testable offline."""
from __future__ import annotations

import os
import threading
from concurrent.futures import ProcessPoolExecutor
from typing import Optional

_worker_tok = None


class ByteTokenizer:
    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = vocab_size
        self.eos_token_id = None

    def encode(self, text: str) -> list:
        return [b % self.vocab_size for b in text.encode("utf-8")] or [0]

    def decode(self, ids) -> str:
        return bytes(int(i) % 256 for i in ids).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, add_generation_prompt=True) -> str:
        return "".join(f"<{m.get('role', 'user')}>{m.get('content', '')}" for m in messages) + ("<assistant>" if add_generation_prompt else "")


def load_tokenizer(path: Optional[str], vocab_size: int = 1024):
    if path and os.path.isdir(path):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(path, trust_remote_code=False)
    return ByteTokenizer(vocab_size)


def _init_worker(path, vocab_size, cores):
    global _worker_tok
    if cores and hasattr(os, "sched_setaffinity"):
        try:
            os.sched_setaffinity(0, cores)
        except OSError:
            pass
    _worker_tok = load_tokenizer(path, vocab_size)


def _encode(text):
    return list(_worker_tok.encode(text))


class TokenizerPool:
    def __init__(self, path: Optional[str] = None, vocab_size: int = 1024, workers: Optional[int] = None,
                 threshold: Optional[int] = None, affinity: Optional[str] = None, enabled: Optional[bool] = None):
        self.tokenizer = load_tokenizer(path, vocab_size)
        self.enabled = os.environ.get("TOKENIZER_PROC_POOL", "0") == "1" if enabled is None else enabled
        self.threshold = int(os.environ.get("TOKENIZER_PROC_POOL_THRES", "2048")) if threshold is None else threshold
        n = int(os.environ.get("TOKENIZER_WORKER_NUM", "4")) if workers is None else workers
        aff = os.environ.get("TOKENIZER_AFFINITY_CORES", "") if affinity is None else affinity
        cores = self._parse_cores(aff)
        self._pool_args = (n, path, vocab_size, cores)
        self.pool_restarts = 0
        self._replace_lock = threading.Lock()
        self.pool = self._new_pool() if self.enabled else None

    def _new_pool(self) -> ProcessPoolExecutor:
        n, path, vocab_size, cores = self._pool_args
        return ProcessPoolExecutor(n, initializer=_init_worker, initargs=(path, vocab_size, cores))

    @staticmethod
    def _parse_cores(spec: str) -> set:
        cores = set()
        for part in filter(None, spec.split(",")):
            if "-" in part:
                a, b = part.split("-")
                cores |= set(range(int(a), int(b) + 1))
            else:
                cores.add(int(part))
        return cores

    def encode(self, text: str) -> list:
        if self.pool is not None and len(text) >= self.threshold:
            from concurrent.futures.process import BrokenProcessPool
            pool = self.pool
            try:
                return pool.submit(_encode, text).result()
            except BrokenProcessPool:
                # a worker died (killed for memory, say): every later submit would fail too.  This prompt is tokenised
                # here, and the pool is replaced for the next ones (once, however many threads notice).
                with self._replace_lock:
                    if self.pool is pool:
                        try:
                            pool.shutdown(wait=False, cancel_futures=True)
                        finally:
                            self.pool = self._new_pool()
                            self.pool_restarts += 1
        return list(self.tokenizer.encode(text))

    def decode(self, ids) -> str:
        return self.tokenizer.decode(ids)

    def shutdown(self):
        if self.pool is not None:
            self.pool.shutdown(wait=False, cancel_futures=True)
