"""Small per-rank state directory that lets a restart come up with the shapes of the previous run.

The reference persists the KV block count per rank beside its on-disk graph cache so that a restart re-uses the same
shapes (omni/adaptors/vllm/worker/npu_worker.py:166-214, omni/adaptors/vllm/utils.py:169-229), and keeps placement
patterns as ``.npy`` files.  CUDA graphs are re-captured at start here (seconds, not minutes), so what is worth
keeping is what decides their shapes and what took time to learn:

  ``num_kv_blocks``        the block count the memory profile arrived at (a restart skips the profile run)
  ``graph_buckets``        the decode batch sizes that were captured
  ``placement_pattern``    the expert placement in force, ``[world, layers, experts]`` 0/1 (``.npy`` beside the JSON)
  ``placement_ema``        the balancer's moving average of position loads (``.npy``)

A state file is only honoured when its fingerprint (model, dtype, parallel sizes, block size, context length, memory
fraction) equals the running configuration's: anything else would restore shapes of a different deployment.
Writes are atomic (temporary file + rename), one file per rank.
"""
from __future__ import annotations

import json
import logging
import os
import tempfile
from typing import Optional

import numpy as np

logger = logging.getLogger("omni_infer_b200.state_dir")
VERSION = 1


def fingerprint(model_cfg, engine_cfg, world: int = 1) -> dict:
    g = lambda o, k, d=None: getattr(o, k, d)
    return {"version": VERSION, "model": g(model_cfg, "name") or g(engine_cfg, "model"),
            "architecture": g(model_cfg, "architecture"), "layers": g(model_cfg, "num_hidden_layers"),
            "hidden": g(model_cfg, "hidden_size"), "experts": g(model_cfg, "n_routed_experts", 0),
            "quantization": g(model_cfg, "quantization", "none"), "dtype": str(g(model_cfg, "dtype", "")),
            "world": int(world), "tp": g(engine_cfg, "tp_size", 1), "pp": g(engine_cfg, "pp_size", 1),
            "block_size": g(engine_cfg, "block_size"), "max_model_len": g(engine_cfg, "max_model_len"),
            "max_num_seqs": g(engine_cfg, "max_num_seqs"), "gpu_memory_utilization": g(engine_cfg, "gpu_memory_utilization", None),
            "num_speculative_tokens": g(engine_cfg, "num_speculative_tokens", 0),
            # options that change what a rank holds (K/V heads, vocabulary rows, expert slots, window pool)
            "attn_tp": bool(g(engine_cfg, "attn_tp", False)), "vocab_parallel": bool(g(engine_cfg, "vocab_parallel", False)),
            "shared_expert_ranks": int(g(engine_cfg, "shared_expert_ranks", 0) or 0),
            "omni_attn": bool(g(engine_cfg, "enable_omni_attn", False))}


class StateDir:
    def __init__(self, path: str, rank: int, fp: dict):
        self.path, self.rank, self.fp = path, int(rank), fp
        os.makedirs(path, exist_ok=True)
        self._cache: Optional[dict] = None

    # ------------------------------------------------------------------ files
    def _json(self) -> str:
        return os.path.join(self.path, f"state_rank{self.rank}.json")

    def _npy(self, key: str) -> str:
        return os.path.join(self.path, f"{key}_rank{self.rank}.npy")

    def _atomic(self, final: str, write) -> None:
        fd, tmp = tempfile.mkstemp(dir=self.path, prefix=".tmp_", suffix=os.path.basename(final))
        try:
            with os.fdopen(fd, "wb") as f:
                write(f)
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, final)
        except BaseException:
            if os.path.exists(tmp):
                os.unlink(tmp)
            raise

    # ------------------------------------------------------------------ read
    def load(self) -> dict:
        """The saved fields, or {} when there is no file, it cannot be read, or it belongs to another configuration."""
        if self._cache is not None:
            return self._cache
        self._cache = {}
        try:
            with open(self._json()) as f:
                data = json.load(f)
        except FileNotFoundError:
            return self._cache
        except (OSError, json.JSONDecodeError) as e:
            logger.warning("state file %s is unreadable (%s): starting cold", self._json(), e)
            return self._cache
        if data.get("fingerprint") != self.fp:
            diff = sorted(k for k in set(self.fp) | set(data.get("fingerprint", {}))
                          if self.fp.get(k) != data.get("fingerprint", {}).get(k))
            logger.info("state file %s belongs to another configuration (differs in %s): starting cold", self._json(), diff)
            return self._cache
        self._cache = dict(data.get("fields", {}))
        return self._cache

    def get(self, key: str, default=None):
        return self.load().get(key, default)

    def get_array(self, key: str) -> Optional[np.ndarray]:
        if not self.load().get(key):
            return None
        try:
            return np.load(self._npy(key))
        except (OSError, ValueError) as e:
            logger.warning("saved array %s is unreadable (%s)", self._npy(key), e)
            return None

    # ------------------------------------------------------------------ write
    def save(self, **fields) -> None:
        cur = dict(self.load())
        for k, v in fields.items():
            if isinstance(v, np.ndarray):
                self._atomic(self._npy(k), lambda f, a=v: np.save(f, a))
                cur[k] = True
            else:
                cur[k] = v
        blob = json.dumps({"fingerprint": self.fp, "fields": cur}, indent=1).encode()
        self._atomic(self._json(), lambda f: f.write(blob))
        self._cache = cur
