"""Pipeline-parallel plumbing: layer ranges per stage, hidden-state hand-over between stages on point-to-point
sends (NCCL p2p on GPUs, gloo on CPU ranks), and the token broadcast from the last stage.

The reference inherits its host engine's pipeline groups and keeps the model-side plumbing (missing-layer
placeholders, intermediate tensors) without any hardware-specific scheduling
(omni/adaptors/vllm/distributed/parallel_state.py:141-186, omni/models/deepseek/deepseek_v3.py:786,
omni/models/qwen/qwen2.py:482).  The same surface here: world ranks are laid out ``[pp][inner]``; stage ``s`` owns a
contiguous block of decoder layers, the first stage embeds, the last stage applies the final norm, computes logits
and samples, and broadcasts the sampled tokens so that every stage's scheduler advances identically (all stages of
a pipeline are given the same requests).  Sends are asynchronous: a stage posts its send and goes on to the next
step's host work; the handles are reaped before the buffers are reused."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from .parallel_state import get_parallel_state


class PPMissingLayer(nn.Module):
    """Placeholder for a decoder layer that lives on another stage (keeps layer indices and parameter names)."""

    def forward(self, *args, **kwargs):
        raise RuntimeError("this layer belongs to another pipeline stage")


def layer_range(num_layers: int, pp_rank: int, pp_size: int) -> tuple:
    """Contiguous, as even as possible; the remainder goes to the middle stages first (the first stage also holds
    the embedding, the last one the LM head)."""
    base, rem = divmod(num_layers, pp_size)
    sizes = [base] * pp_size
    order = sorted(range(pp_size), key=lambda s: (s in (0, pp_size - 1), s))
    for s in order[:rem]:
        sizes[s] += 1
    lo = sum(sizes[:pp_rank])
    return lo, lo + sizes[pp_rank]


class PipelineStage:
    def __init__(self):
        ps = get_parallel_state()
        self.size, self.rank = ps.pp_size, ps.pp_rank
        self.group = ps.group("pp") if self.size > 1 else None
        self._pending: list = []

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.size - 1

    def _peer(self, stage: int) -> int:
        return self.group.ranks[stage]

    def reap(self) -> None:
        for w, _keep in self._pending:
            w.wait()
        self._pending = []

    def send_intermediate(self, h: torch.Tensor, residual: torch.Tensor) -> None:
        """Post the hand-over of (hidden, residual) to the next stage; returns at once."""
        self.reap()
        buf = torch.stack([h, residual], 0).contiguous()
        w = dist.isend(buf, dst=self._peer(self.rank + 1), group=self.group.group)
        self._pending.append((w, buf))

    def recv_intermediate(self, rows: int, hidden: int, dtype, device):
        buf = torch.empty(2, rows, hidden, dtype=dtype, device=device)
        dist.recv(buf, src=self._peer(self.rank - 1), group=self.group.group)
        return buf[0], buf[1]

    def broadcast_tokens(self, toks: Optional[torch.Tensor], n: int, device) -> torch.Tensor:
        """Sampled token ids of the last stage, on every stage."""
        if self.size == 1:
            return toks
        if toks is None:
            toks = torch.empty(n, dtype=torch.int64, device=device)
        dist.broadcast(toks, src=self._peer(self.size - 1), group=self.group.group)
        return toks
