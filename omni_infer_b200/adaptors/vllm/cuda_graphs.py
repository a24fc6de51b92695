"""CUDA-graph buckets for decode steps.

The reference compiles one vendor graph per decode "gear" (padded batch size) and dispatches on
``input_ids.shape[0]`` (omni/adaptors/vllm/compilation/wrapper.py:30-88,
omni/adaptors/vllm/compilation/compile_config.py:91-111).  Here every gear is a captured CUDA graph over
static input buffers: a step copies its inputs into the buffers and replays; the kernels read counts,
slots and the expert selector from device memory, so one graph serves every batch of that bucket."""
from __future__ import annotations

import torch

from ...layers.common import AttnMetadata
from ...ops import _native as nat


class DecodeGraphs:
    def __init__(self, runner):
        self.r = runner
        self.graphs: dict = {}
        self.pool = None

    def has(self, padded: int) -> bool:
        return padded in self.graphs

    def _static_inputs(self, padded: int):
        r = self.r
        dev, tpr = r.device, r.tpr
        n = padded * tpr
        md = AttnMetadata(
            is_prefill=False,
            positions=torch.zeros(n, dtype=torch.int64, device=dev),
            slot_mapping=torch.full((n,), -1, dtype=torch.int64, device=dev),
            block_table=torch.zeros(padded, r._bt_width, dtype=torch.int32, device=dev),
            seq_lens=torch.zeros(padded, dtype=torch.int32, device=dev),
            tokens_per_req=tpr,
            q_seq_lens=torch.zeros(n, dtype=torch.int32, device=dev),
            q_to_seq=(torch.arange(n, dtype=torch.int32, device=dev) // tpr).int(),
            max_seq_len=r.cfg.max_model_len,
            num_valid=torch.zeros(1, dtype=torch.int32, device=dev))
        ids = torch.zeros(n, dtype=torch.int64, device=dev)
        return ids, md

    def capture(self, padded: int) -> None:
        r = self.r
        ids, md = self._static_inputs(padded)
        r._agree_ep_path(padded * r.tpr, 1, False)
        # warm-up on a side stream (first-use set-up such as shared-memory attributes must not be captured)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                h = r.model(ids, md, r.kv_caches)
                r.model.compute_logits(h)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = nat.launch_count()
        with torch.cuda.graph(g, pool=self.pool):
            hidden = r.model(ids, md, r.kv_caches)
            logits = r.model.compute_logits(hidden)
        captured = nat.launch_count() - before
        nat.add_launches(-captured)          # capture itself runs nothing
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[padded] = (g, ids, md, hidden, logits, captured)

    def replay(self, padded: int, ids: torch.Tensor, md: AttnMetadata):
        g, s_ids, s_md, hidden, logits, captured = self.graphs[padded]
        s_ids.copy_(ids)
        s_md.positions.copy_(md.positions)
        s_md.slot_mapping.copy_(md.slot_mapping)
        s_md.block_table.copy_(md.block_table)
        s_md.seq_lens.copy_(md.seq_lens)
        s_md.q_seq_lens.copy_(md.q_seq_lens)
        if md.num_valid is not None:
            s_md.num_valid.copy_(md.num_valid)
        else:
            s_md.num_valid.fill_(padded * self.r.tpr)
        g.replay()
        nat.add_launches(captured)
        return hidden, logits
