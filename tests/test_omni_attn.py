"""Omni-Attention: ring-window arithmetic, the two-pool manager, transfer block selection, and engine runs in
which short sequences (that fit the window) decode exactly as without compression."""
import torch

from omni_infer_b200 import ops
from omni_infer_b200.accelerators.cache import (OmniAttentionSpec, OmniAttnConfig, OmniAttnState, OmniKVCacheManager,
                                                compute_omni_attn_metadata_ref, default_pattern)
from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
from omni_infer_b200.engine.request import Request, SamplingParams


def test_ring_window_positions():
    bs, sink, recent = 16, 1, 3
    cap = 64
    # sequence that started short: linear until the capacity, then wraps inside [16, 64)
    seen = []
    for L in range(1, 200):
        pos, eff = compute_omni_attn_metadata_ref(L, 10, bs, sink, recent)
        assert 0 <= pos < cap and eff == min(L, cap)
        if L > cap:
            assert pos >= sink * bs
        seen.append(pos)
    assert seen[:64] == list(range(64))
    assert seen[64:64 + 48] == list(range(16, 64))          # one full turn of the ring
    # long prompt: the first generated token takes the oldest window entry
    assert compute_omni_attn_metadata_ref(101, 100, bs, sink, recent)[0] == 16
    sl = torch.tensor([5, 64, 65, 101, 0], dtype=torch.int32)
    pl = torch.tensor([3, 10, 10, 100, 0], dtype=torch.int32)
    bt = torch.arange(20, dtype=torch.int32).view(5, 4)
    slots, eff = ops.omni_attn_slots(sl, pl, bt, bs, sink, recent)
    for b in range(4):
        pos, e = compute_omni_attn_metadata_ref(int(sl[b]), int(pl[b]), bs, sink, recent)
        assert int(slots[b]) == int(bt[b, pos // bs]) * bs + pos % bs and int(eff[b]) == e
    assert int(slots[4]) == -1


def test_two_pool_manager_and_prefill_slots():
    spec = OmniAttentionSpec(16, 1, 3)
    m = OmniKVCacheManager(32, 16, spec, num_window_blocks=9)       # room for two windows
    reqs = [Request(f"r{i}", list(range(100))) for i in range(3)]
    assert m.allocate_slots(reqs[0], 100) is not None and len(reqs[0].omni_block_ids) == 4
    assert m.allocate_slots(reqs[1], 100) is not None
    assert m.allocate_slots(reqs[2], 100) is None                    # no window left: nothing allocated
    assert reqs[2].block_ids == []
    m.free(reqs[0])
    assert m.allocate_slots(reqs[2], 100) is not None
    st = OmniAttnState(OmniAttnConfig(1, 3, 0.2, [0, 1]), 16)
    slots = st.prefill_slots([5, 6, 7, 8], 0, 100, 100)
    assert slots[:16] == [5 * 16 + i for i in range(16)]             # sink
    assert all(s == -1 for s in slots[16:52])                        # middle of the prompt is not kept
    assert slots[52] == 6 * 16 and slots[99] == 8 * 16 + 15          # last 48 tokens fill the window in order
    pairs = st.select_transfer_blocks(list(range(10, 17)), 100, [5, 6, 7, 8])
    assert pairs == [(10, 5), (14, 6), (15, 7), (16, 8)]
    assert default_pattern(10, 0.2)[:2] == [0, 0] and sum(default_pattern(61, 0.2)) > 40


def test_engine_with_omni_attention():
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]

    def run(omni, max_tokens, prompts_):
        kw = dict(enable_omni_attn=True, omni_attn_config={"sink": 1, "recent": 3, "pattern": [0, 1]}) if omni else {}
        e = EngineCore(EngineConfig(block_size=16, num_kv_blocks=64, max_model_len=256, device="cpu", max_num_seqs=4, **kw))
        ids = [e.add_request(p, SamplingParams(max_tokens=max_tokens)) for p in prompts_]
        outs = e.run_until_done()
        return [outs[i] for i in ids], e

    base, _ = run(False, 30, prompts)
    got, eng = run(True, 30, prompts)
    assert got == base                                   # 50 tokens fit the 64-token window: identical
    assert eng.kv.window_free and len(eng.kv.window_free) == 4 * 4
    # beyond the window the compressed layer forgets the middle: still runs, output may differ
    long_out, _ = run(True, 80, prompts[:1])
    assert len(long_out[0]) == 80
