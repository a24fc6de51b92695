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


def test_window_holds_sink_and_most_recent_tokens_whatever_the_history():
    """Replay of the writes into one request's window (64 entries: 16 sink + 48 recent): prefill of any prompt length,
    decode steps, and a recompute after a preemption (prompt + generated tokens in one or several prefill chunks).  At
    every point the window must hold the first 16 tokens and the most recent ones, each exactly once."""
    import random
    bs, sink, recent = 16, 1, 3
    st_, rt, cap = 16, 48, 64
    state = OmniAttnState(OmniAttnConfig(sink, recent, 0.2, [0, 1]), bs)
    blocks = [7, 3, 9, 5]                                   # window blocks in any order

    def where(slot):
        return blocks.index(slot // bs) * bs + slot % bs

    def expect(window, L):
        held = sorted(v for v in window if v is not None)
        want = list(range(L)) if L <= cap else list(range(st_)) + list(range(L - rt, L))
        assert held == want, (L, held[:20], want[:20])

    rnd = random.Random(3)
    for prompt_len in [1, 5, 16, 17, 63, 64, 65, 80, 111, 112, 113, 200]:
        for n_gen_before_preempt in [0, 1, 7, 49, 130]:
            window = [None] * cap
            # ---- first life: prefill the prompt (in two chunks), then decode
            cut = rnd.randint(0, prompt_len)
            for start, n in ((0, cut), (cut, prompt_len - cut)):
                for i, s in enumerate(state.prefill_slots(blocks, start, n, prompt_len)):
                    if s >= 0:
                        window[where(s)] = start + i
            expect(window, prompt_len)
            L = prompt_len
            for _ in range(n_gen_before_preempt):
                L += 1
                pos, eff = compute_omni_attn_metadata_ref(L, prompt_len, bs, sink, recent)
                window[pos] = L - 1
                assert eff == min(L, cap)
                expect(window, L)
            # ---- preempted: the window is lost; prompt + generated tokens are prefilled again, in chunks
            redo = [None] * cap
            total = L
            pieces, at = [], 0
            while at < total:
                n = rnd.randint(1, max(1, total // 2))
                pieces.append((at, min(n, total - at)))
                at += pieces[-1][1]
            rnd.shuffle(pieces)                              # a scatter has no order: neither may the result depend on it
            for start, n in pieces:
                slots = state.prefill_slots(blocks, start, n, prompt_len, total_len=total)
                assert len(slots) == n
                for i, s in enumerate(slots):
                    if s >= 0:
                        assert redo[where(s)] is None, "two tokens of one prefill were sent to the same window entry"
                        redo[where(s)] = start + i
            assert redo == window, (prompt_len, n_gen_before_preempt)
            # ---- and decoding goes on from there
            for _ in range(60):
                L += 1
                pos, _ = compute_omni_attn_metadata_ref(L, prompt_len, bs, sink, recent)
                redo[pos] = L - 1
                expect(redo, L)


def test_engine_with_omni_attention_survives_preemption():
    """A KV pool so small that running requests are preempted and recomputed while Omni-Attention is on and the
    sequences (80 tokens) have outgrown the 64-token window: the recompute rebuilds the window as the decode steps had
    left it, so the tokens equal those of a run that never preempts."""
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (20,), generator=g).tolist() for _ in range(3)]

    def run(num_blocks):
        e = EngineCore(EngineConfig(block_size=16, num_kv_blocks=num_blocks, max_model_len=256, device="cpu", max_num_seqs=4,
                                    enable_omni_attn=True, omni_attn_config={"sink": 1, "recent": 3, "pattern": [0, 1]}))
        ids = [e.add_request(p, SamplingParams(max_tokens=60)) for p in prompts]
        outs = e.run_until_done()
        return [outs[i] for i in ids], e

    roomy, _ = run(64)
    tight, eng = run(13)                                    # 12 usable blocks for 3 x 80 tokens: somebody has to go
    assert eng.scheduler.stats["preemptions"] > 0
    assert tight == roomy


def test_omni_attention_with_multi_step_rounds_and_async_scheduling():
    """Several model steps per scheduling round: the windows of the compressed layers have to move on with every step of
    the round, not once per round.  Sequences grow past the window; tokens equal the one-step-per-round run."""
    import pytest
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 61, 90)]
    omni = dict(enable_omni_attn=True, omni_attn_config={"sink": 1, "recent": 2, "pattern": [1, 0]})

    def run(**kw):
        e = EngineCore(EngineConfig(block_size=16, num_kv_blocks=64, max_model_len=256, device="cpu", max_num_seqs=4, **omni, **kw))
        ids = [e.add_request(p, SamplingParams(max_tokens=40)) for p in prompts]
        outs = e.run_until_done()
        return [outs[i] for i in ids]

    want = run()
    assert run(num_step=3) == want
    assert run(num_step=2, async_schedule=True) == want
    # what cannot be combined is refused at start, not discovered as an index error later
    for bad in (dict(enable_chunked_prefill=True), dict(enable_prefix_caching=True)):
        with pytest.raises(ValueError):
            EngineCore(EngineConfig(block_size=16, num_kv_blocks=64, max_model_len=256, device="cpu", **omni, **bad))
