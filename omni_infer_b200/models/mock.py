"""Mock model factory for integration tests without real weights or without a GPU
(reference: omni/models/mock/mock.py, tests/test_framework/vllm_mock/README.md:15-88).

``mock_model_class_factory(base)`` wraps any model class.  Modes, selected by environment variables:
  RANDOM_MODE    random hidden states / logits of the right shapes (optionally sleeping FORWARD_TIME ms)
  CAPTURE_MODE   runs the real model and appends {prompt ids -> sampled ids} to a JSONL file
                 (MOCK_CAPTURE_DIR / MOCK_CAPTURE_FILE)
  REPLAY_MODE    serves the captured tokens keyed by the prompt ids (SIMULATE_ELAPSED_TIME replays the recorded
                 step latency)
  KV_CACHE_MODE  additionally fills the KV cache slots of the step with random values so PD transfers move data
  NO_GPU_MOCK    the whole stack runs on CPU
The wrapper keeps the model interface (forward -> hidden states, compute_logits)."""
from __future__ import annotations

import json
import os
import time
from pathlib import Path

import torch


def _capture_path() -> Path:
    d = Path(os.environ.get("MOCK_CAPTURE_DIR", "/tmp/omni_mock"))
    d.mkdir(parents=True, exist_ok=True)
    return d / os.environ.get("MOCK_CAPTURE_FILE", "capture.jsonl")


class ReplayStore:
    """prompt-prefix -> next token table built from a capture file."""

    def __init__(self, path: Path):
        self.table = {}
        if path.exists():
            for line in path.read_text().splitlines():
                rec = json.loads(line)
                seq = rec["prompt"] + rec["output"]
                for i in range(len(rec["prompt"]), len(seq)):
                    self.table[tuple(seq[:i])] = (seq[i], rec.get("step_ms", 0.0))

    def next_token(self, prefix):
        return self.table.get(tuple(prefix), (0, 0.0))


def mock_model_class_factory(base_cls):
    class MockModel(base_cls):
        mock_base = base_cls

        def __init__(self, cfg, **kw):
            self.random_mode = os.environ.get("RANDOM_MODE") == "1"
            self.capture_mode = os.environ.get("CAPTURE_MODE") == "1"
            self.replay_mode = os.environ.get("REPLAY_MODE") == "1"
            self.kv_cache_mode = os.environ.get("KV_CACHE_MODE") == "1"
            self.forward_time_ms = float(os.environ.get("FORWARD_TIME", "0"))
            self.simulate_elapsed = os.environ.get("SIMULATE_ELAPSED_TIME") == "1"
            if self.random_mode or self.replay_mode:
                # no real layers needed: keep only what the interface requires
                torch.nn.Module.__init__(self)
                self.cfg = cfg
                self._device = kw.get("device") or "cpu"
                self._dummy = torch.nn.Parameter(torch.zeros(1, device=self._device), requires_grad=False)
                self.is_mla = cfg.use_mla
                self._num_layers = cfg.num_hidden_layers
                self._gen = torch.Generator(device="cpu").manual_seed(0)
                self._replay = ReplayStore(_capture_path()) if self.replay_mode else None
                self._pending_tokens = None
            else:
                super().__init__(cfg, **kw)
            self._cap_prompts = {}

        # ---- interface
        @property
        def num_kv_layers(self):
            if self.random_mode or self.replay_mode:
                return self._num_layers
            return super().num_kv_layers

        def process_weights_after_loading(self):
            if not (self.random_mode or self.replay_mode):
                super().process_weights_after_loading()

        def should_use_eager_mode(self, md):
            return True

        def forward(self, input_ids, md, kv_caches, inputs_embeds=None):
            if self.forward_time_ms > 0:
                time.sleep(self.forward_time_ms / 1e3)
            if not (self.random_mode or self.replay_mode):
                return super().forward(input_ids, md, kv_caches, inputs_embeds)
            T = input_ids.shape[0]
            if self.kv_cache_mode:
                ok = md.slot_mapping >= 0
                for c in kv_caches:
                    for t in (c if isinstance(c, (tuple, list)) else (c,)):
                        flat = t.view(-1, *t.shape[2:])
                        flat[md.slot_mapping[ok]] = torch.randn(int(ok.sum()), *flat.shape[1:], generator=self._gen).to(flat)
            self._last_ids, self._last_md = input_ids, md
            h = torch.randn(T, self.cfg.hidden_size, generator=self._gen).to(self._dummy.device)
            return h

        def compute_logits(self, hidden):
            if not (self.random_mode or self.replay_mode):
                return super().compute_logits(hidden)
            n, V = hidden.shape[0], self.cfg.vocab_size
            if self.replay_mode and getattr(self, "_replay_prefixes", None):
                logits = torch.full((n, V), -1e4)
                for i, prefix in enumerate(self._replay_prefixes[:n]):
                    tok, ms = self._replay.next_token(prefix)
                    logits[i, tok] = 1e4
                    if self.simulate_elapsed and ms:
                        time.sleep(ms / 1e3)
                return logits.to(hidden.device)
            return torch.randn(n, V, generator=self._gen).to(hidden.device)

        def set_replay_prefixes(self, prefixes):
            """The runner tells the replay model which token prefixes the rows of the next logits belong to."""
            self._replay_prefixes = prefixes

        def load_weights(self, weights, planner=None):
            if self.random_mode or self.replay_mode:
                return set()
            return super().load_weights(weights, planner)

    MockModel.__name__ = "Mock" + base_cls.__name__
    return MockModel


def capture_outputs(prompts, outputs, step_ms: float = 0.0) -> None:
    """Append one JSONL record per request to the capture file (CAPTURE_MODE)."""
    with open(_capture_path(), "a") as f:
        for p, o in zip(prompts, outputs):
            f.write(json.dumps({"prompt": list(p), "output": list(o), "step_ms": step_ms}) + "\n")
