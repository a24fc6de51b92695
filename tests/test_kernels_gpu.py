"""Row / routing / sampling kernels and MLA decode attention vs the fp32 PyTorch references."""
import math

import pytest
import torch

from omni_infer_b200 import ops
from omni_infer_b200.ops import attention as A
from omni_infer_b200.ops import basic as B
from omni_infer_b200.ops import moe as M
from omni_infer_b200.ops import sampling as S

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, rtol=2e-2, atol=2e-2):
    torch.testing.assert_close(a.float(), b.float(), rtol=rtol, atol=atol)


@pytest.mark.parametrize("T,H", [(1, 256), (7, 2048), (33, 7168), (5, 1536)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(T, H, with_res):
    torch.manual_seed(0)
    x = torch.randn(T, H, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    r1 = torch.randn(T, H, device=DEV).bfloat16() if with_res else None
    r2 = r1.clone() if with_res else None
    y = B.rmsnorm(x, w, 1e-6, residual=r1)
    ref = B.rmsnorm_ref(x, w, 1e-6, residual=r2)
    _close(y, ref)
    if with_res:
        _close(r1, r2, 1e-2, 1e-2)


def test_rmsnorm_quant():
    torch.manual_seed(1)
    T, H = 19, 2048
    x = torch.randn(T, H, device=DEV).bfloat16()
    w = torch.ones(H, device=DEV).bfloat16()
    y, q, s = B.rmsnorm(x, w, 1e-6, quant=True)
    deq = ops.dequant_act_ref(q, s)
    assert ((deq - y.float()).abs().max() / y.float().abs().max()).item() < 0.07


def test_quant_fp8_block():
    torch.manual_seed(2)
    x = (torch.randn(37, 1536, device=DEV) * 3).bfloat16()
    q, s = B.quant_fp8_block(x)
    qr, sr = ops.quant_fp8_block_ref(x, ld=s.shape[1])
    _close(s[:, :37], sr[:, :37], 1e-5, 1e-8)
    assert (ops.dequant_act_ref(q, s) - ops.dequant_act_ref(qr, sr)).abs().max().item() < 0.3


def test_silu_mul():
    x = torch.randn(13, 2 * 1408, device=DEV).bfloat16()
    _close(B.silu_mul(x), B.silu_mul_ref(x))


def test_mla_kv_rope_cache():
    torch.manual_seed(3)
    T, heads = 11, 16
    latent = torch.randn(T, 576, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(512, device=DEV)).bfloat16()
    cs = B.rope_cos_sin_table(64, 512, device=DEV)
    pos = torch.randint(0, 512, (T,), device=DEV)
    slots = torch.randperm(64, device=DEV)[:T].long()
    slots[3] = -1
    q1 = torch.randn(T, heads, 192, device=DEV).bfloat16()
    q2 = q1.clone()
    c1 = torch.zeros(4, 16, 576, device=DEV, dtype=torch.bfloat16)
    c2 = c1.clone()
    lat = B.mla_kv_rope_cache(latent, w, 1e-6, cs, pos, slots, c1, q=q1, q_rope_off=128, want_latent=True)
    ref = B.mla_kv_rope_cache_ref(latent, w, 1e-6, cs, pos, slots, c2, q=q2, q_rope_off=128)
    _close(c1, c2)
    _close(q1, q2)
    _close(lat, ref)


@pytest.mark.parametrize("qk_norm", [False, True])
def test_rope_qk_cache(qk_norm):
    torch.manual_seed(4)
    T, hq, hkv, D = 9, 8, 2, 128
    qkv1 = torch.randn(T, (hq + 2 * hkv) * D, device=DEV).bfloat16()
    qkv2 = qkv1.clone()
    cs = B.rope_cos_sin_table(D, 300, base=1e6, device=DEV)
    pos = torch.randint(0, 300, (T,), device=DEV)
    slots = torch.randperm(48, device=DEV)[:T].long()
    kc1 = torch.zeros(3, 16, hkv, D, device=DEV, dtype=torch.bfloat16)
    vc1 = torch.zeros_like(kc1)
    kc2, vc2 = kc1.clone(), vc1.clone()
    qn = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if qk_norm else None
    kn = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if qk_norm else None
    B.rope_qk_cache(qkv1, hq, hkv, D, cs, pos, slots, kc1, vc1, qn, kn)
    B.rope_qk_cache_ref(qkv2, hq, hkv, D, cs, pos, slots, kc2, vc2, qn, kn)
    _close(qkv1, qkv2, 3e-2, 3e-2)
    _close(kc1, kc2, 3e-2, 3e-2)
    _close(vc1, vc2)


def test_embedding():
    table = torch.randn(100, 256, device=DEV).bfloat16()
    ids = torch.tensor([0, 5, 99, 120, 40], device=DEV)
    out = B.embedding(ids, table, vocab_start=0)
    assert torch.equal(out[:3], table[ids[:3]]) and out[3].abs().sum() == 0
    out2 = B.embedding(ids, table[:50], vocab_start=40)
    assert torch.equal(out2[4], table[0]) and out2[0].abs().sum() == 0


@pytest.mark.parametrize("cfg", [
    dict(E=64, k=6, mode="softmax"),
    dict(E=128, k=8, mode="softmax", renorm=True),
    dict(E=256, k=8, mode="sigmoid", bias=True, n_group=8, topk_group=4, group_mode="top2sum", renorm=True, scale=2.5),
    dict(E=8, k=2, mode="softmax"),
    dict(E=160, k=6, mode="softmax", n_group=8, topk_group=3, group_mode="max", scale=16.0),
])
def test_router_topk(cfg):
    torch.manual_seed(5)
    T, E, k = 37, cfg["E"], cfg["k"]
    logits = torch.randn(T, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.1 if cfg.get("bias") else None
    sel = torch.randperm(E + 8, device=DEV)[:E].int()
    counts = torch.zeros(E + 8, dtype=torch.int64, device=DEV)
    kw = dict(mode=cfg["mode"], bias=bias, n_group=cfg.get("n_group", 1), topk_group=cfg.get("topk_group", 1),
              group_mode=cfg.get("group_mode", "max"), renorm=cfg.get("renorm", False), scale=cfg.get("scale", 1.0),
              selector=sel)
    ids, w = M.router_topk(logits, k, counts=counts, **kw)
    rid, rw = M.router_topk_ref(logits, k, **kw)
    assert torch.equal(ids.sort(dim=-1).values, rid.sort(dim=-1).values)
    order, rorder = ids.argsort(dim=-1), rid.argsort(dim=-1)
    _close(w.gather(1, order), rw.gather(1, rorder), 1e-4, 1e-6)
    assert torch.equal(counts, torch.bincount(rid.flatten().long(), minlength=E + 8))


def test_router_forced_balance_and_padding():
    T, E, k = 16, 64, 4
    logits = torch.randn(T, E, device=DEV)
    nv = torch.tensor([10], dtype=torch.int32, device=DEV)
    ids, w = M.router_topk(logits, k, forced_balance=True, num_valid=nv)
    assert (ids[10:] == -1).all() and (w[10:] == 0).all()
    assert torch.equal(ids[:10].flatten().cpu(), (torch.arange(40) % E).int())


@pytest.mark.parametrize("quant", [False, True])
def test_moe_permute_combine(quant):
    torch.manual_seed(6)
    T, H, E, k = 29, 256, 16, 4
    x = torch.randn(T, H, device=DEV).bfloat16()
    ids, w = M.router_topk(torch.randn(T, E, device=DEV), k, renorm=True)
    e_lo, e_local = 4, 8
    perm = M.moe_permute(x, ids, w, e_lo, e_local, quant=quant)
    lens = perm.seg_len.tolist()
    flat = ids.flatten().long() - e_lo
    assert lens == torch.bincount(flat[(flat >= 0) & (flat < e_local)], minlength=e_local).tolist()
    starts = perm.seg_start.tolist()
    assert all(s % 16 == 0 for s in starts)
    xs = ops.dequant_act_ref(perm.x, perm.x_scale) if quant else perm.x.float()
    ro = perm.row_of.view(T, k)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j]) - e_lo
            r = int(ro[t, j])
            if 0 <= e < e_local:
                assert starts[e] <= r < starts[e] + lens[e]
                err = (xs[r] - x[t].float()).abs().max().item()
                assert err < (0.3 if quant else 1e-6)
                assert abs(float(perm.row_w[r]) - float(w[t, j])) < 1e-6
            else:
                assert r == -1
    if quant:   # rows that arrive already quantised are copied, not re-quantised: identical bytes and scales
        xq_in = ops.quant_fp8_block(x)
        perm2 = M.moe_permute(x, ids, w, e_lo, e_local, quant=True, xq_in=xq_in)
        assert perm2.seg_len.tolist() == lens and perm2.seg_start.tolist() == starts
        ro2 = perm2.row_of.view(T, k)
        for t_ in range(T):
            for j in range(k):
                r = int(ro2[t_, j])
                if 0 <= int(ids[t_, j]) - e_lo < e_local:
                    assert torch.equal(perm2.x.view(torch.uint8)[r], xq_in[0].view(torch.uint8)[t_])
                    assert torch.equal(perm2.x_scale[:, r], xq_in[1][:, t_])
                    assert abs(float(perm2.row_w[r]) - float(w[t_, j])) < 1e-6
                else:
                    assert r == -1
    y = torch.randn(perm.x.shape[0], H, device=DEV).bfloat16()
    shared = torch.randn(T, H, device=DEV).bfloat16()
    out = M.moe_combine(y, perm.row_of, T, k, w=w, shared=shared)
    _close(out, M.moe_combine_ref(y, perm.row_of, T, k, w=w, shared=shared))


def test_argmax_and_sampling():
    torch.manual_seed(7)
    logits = torch.randn(9, 5000, device=DEV)
    assert torch.equal(S.argmax(logits), logits.argmax(-1))
    assert torch.equal(S.argmax(logits.bfloat16()), logits.bfloat16().float().argmax(-1))
    B_, V = 64, 1000
    lg = torch.randn(B_, V, device=DEV) * 2
    temp = torch.full((B_,), 0.8, device=DEV)
    temp[0] = 0.0
    tk = torch.full((B_,), 20, dtype=torch.int32, device=DEV)
    tp = torch.full((B_,), 0.9, device=DEV)
    u = torch.rand(B_, device=DEV)
    ids = S.sample_topk_topp(lg, temp, tk, tp, u)
    ref = S.sample_topk_topp_ref(lg.cpu(), temp.cpu(), tk.cpu(), tp.cpu(), u.cpu())
    assert ids[0] == lg[0].argmax()
    assert (ids.cpu() == ref).float().mean().item() > 0.9      # threshold ties may move a boundary token
    top20 = lg.topk(20, dim=-1).indices
    assert all(ids[b] in top20[b] for b in range(B_))


def test_mtp_verify_and_step_advance():
    inp = torch.tensor([[5, 7, 9], [1, 2, 3], [4, 4, 4]], device=DEV)
    fwd = torch.tensor([[7, 9, 11], [2, 8, 3], [6, 4, 4]], device=DEV)
    out, acc, last, nxt = S.mtp_verify(inp, fwd)
    ro, ra, rl, rn = S.mtp_verify_ref(inp, fwd)
    assert torch.equal(out, ro) and torch.equal(acc, ra) and torch.equal(last, rl) and torch.equal(nxt, rn)
    assert acc.tolist() == [2, 1, 0]
    bt = torch.arange(12, dtype=torch.int32, device=DEV).view(3, 4)
    seq = torch.tensor([15, 0, 16], dtype=torch.int32, device=DEV)
    pos = torch.zeros(3, dtype=torch.int64, device=DEV)
    slots = torch.zeros(3, dtype=torch.int64, device=DEV)
    S.step_advance(pos, seq, slots, bt, 16)
    assert seq.tolist() == [16, 0, 17] and pos.tolist() == [15, 0, 16]
    assert slots.tolist() == [0 * 16 + 15, 0, 9 * 16 + 0]


def test_omni_attn_slots():
    bs, sink, recent = 16, 1, 3
    seq = torch.tensor([5, 64, 65, 200, 0], dtype=torch.int32, device=DEV)
    prm = torch.tensor([3, 40, 40, 100, 0], dtype=torch.int32, device=DEV)
    bt = torch.arange(20, dtype=torch.int32, device=DEV).view(5, 4)
    s, e = S.omni_attn_slots(seq, prm, bt, bs, sink, recent)
    rs, re = S.omni_attn_slots_ref(seq.cpu(), prm.cpu(), bt.cpu(), bs, sink, recent)
    assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)


@pytest.mark.parametrize("H,lens,bs,splits", [
    (128, [1, 31, 32, 33, 200], 128, 1),
    (16, [77, 500, 128], 64, 1),
    (128, [700, 64], 128, 4),
    (64, [1000], 32, 0),
    (128, [0, 129], 128, 1),
])
def test_mla_decode(H, lens, bs, splits):
    torch.manual_seed(8)
    Bq = len(lens)
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nblocks = Bq * max_blocks + 2
    cache = (torch.randn(nblocks, bs, 576, device=DEV) * 0.5).bfloat16()
    perm = torch.randperm(nblocks - 1, device=DEV)[: Bq * max_blocks].int() + 1
    bt = perm.view(Bq, max_blocks).contiguous()
    q = (torch.randn(Bq, H, 576, device=DEV) * 0.5).bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(192)
    out = A.mla_decode(q, cache, bt, sl, scale, num_splits=splits, max_seq_len=max(lens))
    ref = A.mla_decode_ref(q, cache, bt, sl, scale)
    _close(out, ref, 3e-2, 2e-2)


@pytest.mark.parametrize("q_per_seq,seq_lens,splits", [(2, [300, 65, 1024], 1), (4, [64, 700], 1), (3, [129, 5, 2047], 2),
                                                       (1, [63, 64, 65, 127, 128, 191, 192, 193], 1)])
def test_mla_decode_query_rows_of_one_sequence(q_per_seq, seq_lens, splits):
    """Several q rows per request (a verified token plus MTP drafts): row j of a request sees its length minus the
    rows after it, all rows share one block-table row through q_to_seq; lengths around the 64-token tile edges so that
    both CTAs of a pair get odd and even tile counts."""
    torch.manual_seed(21)
    H, bs = 128, 128
    B_ = len(seq_lens)
    max_blocks = (max(seq_lens) + bs - 1) // bs + 1
    nblocks = B_ * max_blocks + 2
    cache = (torch.randn(nblocks, bs, 576, device=DEV) * 0.5).bfloat16()
    bt = (torch.randperm(nblocks - 1, device=DEV)[: B_ * max_blocks].int() + 1).view(B_, max_blocks).contiguous()
    rows, q2s = [], []
    for i, L in enumerate(seq_lens):
        for j in range(q_per_seq):
            rows.append(max(0, L - (q_per_seq - 1 - j)))
            q2s.append(i)
    Bq = len(rows)
    q = (torch.randn(Bq, H, 576, device=DEV) * 0.5).bfloat16()
    sl = torch.tensor(rows, dtype=torch.int32, device=DEV)
    q2 = torch.tensor(q2s, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(192)
    out = A.mla_decode(q, cache, bt, sl, scale, q_to_seq=q2, num_splits=splits, max_seq_len=max(seq_lens))
    ref = A.mla_decode_ref(q, cache, bt, sl, scale, q_to_seq=q2)
    _close(out, ref, 3e-2, 2e-2)


@pytest.mark.parametrize("pattern", ["late_peak", "early_peak", "alternating"])
def test_mla_decode_wide_score_range(pattern):
    """Scores whose maximum moves by far more than the lazy-rescale threshold between tiles: the late tiles dominate,
    the first tile dominates, or odd and even tiles (computed by different CTAs of a pair) sit at different levels."""
    torch.manual_seed(22)
    H, bs, L = 128, 128, 640
    cache = (torch.randn(8, bs, 576, device=DEV) * 0.3).bfloat16()
    bt = (torch.arange(6, device=DEV, dtype=torch.int32) + 1).view(1, 6)
    q = (torch.randn(1, H, 576, device=DEV) * 0.5).bfloat16()
    flat = cache.view(-1, 576)
    tile = torch.arange(L, device=DEV) // 64
    boost = {"late_peak": (tile >= 8).float() * 6.0, "early_peak": (tile == 0).float() * 6.0,
             "alternating": (tile % 2).float() * 5.0}[pattern]
    # make the keys of the boosted tiles align with q's mean direction, so that their scores are far larger
    direction = q[0].float().mean(0)
    direction = direction / direction.norm()
    slots = (bt[0, torch.arange(L, device=DEV) // bs].long() * bs + torch.arange(L, device=DEV) % bs)
    flat[slots] = (flat[slots].float() + boost[:, None] * direction[None, :] * 30.0).bfloat16()
    sl = torch.tensor([L], dtype=torch.int32, device=DEV)
    scale = 1.0
    out = A.mla_decode(q, cache, bt, sl, scale, num_splits=1, max_seq_len=L)
    ref = A.mla_decode_ref(q, cache, bt, sl, scale)
    _close(out, ref, 3e-2, 2e-2)


@pytest.mark.parametrize("qlens,ctx", [([5, 130, 64], [0, 0, 0]), ([256], [0]), ([17, 100], [40, 0]), ([1, 1], [300, 5])])
def test_fmha_mla_prefill(qlens, ctx):
    """Non-absorbed MLA prefill: q 192 wide, k = kv_b slice | shared roped k_pe, v = kv_b slice."""
    torch.manual_seed(9)
    H, nope, rope, vd = 4, 128, 64, 128
    klens = [q + c for q, c in zip(qlens, ctx)]
    Tq, Tk = sum(qlens), sum(klens)
    q = (torch.randn(Tq, H, nope + rope, device=DEV) * 0.5).bfloat16()
    kv = (torch.randn(Tk, H * (nope + vd), device=DEV) * 0.5).bfloat16()
    lat = (torch.randn(Tk, 576, device=DEV) * 0.5).bfloat16()
    cu_q = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(klens).cumsum(0)), dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(192)
    out = A.mla_prefill(q, kv, lat, H, nope, rope, vd, cu_q, cu_k, scale, max(qlens), max(klens))
    ref = A.mla_prefill_ref(q, kv, lat, H, nope, rope, vd, cu_q, cu_k, scale)
    _close(out, ref, 3e-2, 2e-2)


@pytest.mark.parametrize("qlens", [[9, 200], [128, 1, 77]])
def test_fmha_gqa_prefill(qlens):
    torch.manual_seed(10)
    Hq, Hkv, D = 8, 2, 128
    T = sum(qlens)
    qkv = (torch.randn(T, Hq + 2 * Hkv, D, device=DEV) * 0.5).bfloat16()
    q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    out = A.gqa_prefill(q, k, v, cu, cu, scale, max(qlens), max(qlens))
    ref = A.attn_prefill_ref(q, k, v, cu, cu, scale)
    _close(out, ref, 3e-2, 2e-2)


@pytest.mark.parametrize("lens,splits,Hq,Hkv,bs", [([1, 33, 500], 1, 32, 4, 16), ([2000, 64], 4, 32, 4, 16), ([0, 77], 0, 32, 4, 16),
                                                   ([31, 32, 65, 4100], 0, 32, 2, 128),      # 16 query heads per KV head
                                                   ([300, 129], 3, 8, 4, 128), ([1500], 0, 32, 4, 128)])
def test_gqa_paged_decode(lens, splits, Hq, Hkv, bs):
    torch.manual_seed(11)
    B_, D = len(lens), 128
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nb = B_ * max_blocks + 1
    kc = (torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5).bfloat16()
    vc = (torch.randn(nb, bs, Hkv, D, device=DEV) * 0.5).bfloat16()
    bt = (torch.randperm(nb - 1, device=DEV)[: B_ * max_blocks].int() + 1).view(B_, max_blocks).contiguous()
    q = (torch.randn(B_, Hq, D, device=DEV) * 0.5).bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    from omni_infer_b200.ops.fmha import gqa_paged_decode
    out = gqa_paged_decode(q, kc, vc, bt, sl, scale, max(lens), num_splits=splits)
    ref = A.gqa_decode_ref(q, kc, vc, bt, sl, scale)
    _close(out, ref, 3e-2, 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_apply_penalties(dtype):
    """Repetition / frequency / presence penalties against the fp32 reference; one row is neutral and must be untouched."""
    from omni_infer_b200.ops import sampling as S
    torch.manual_seed(31)
    Bn, V, L = 5, 5000, 300
    logits = (torch.randn(Bn, V, device=DEV) * 3).to(dtype)
    hist = torch.randint(0, V, (Bn, L), device=DEV, dtype=torch.int32)
    hist[:, 250:] = -1
    hist[1, 100:120] = 7                      # a token repeated in the output
    npr = torch.tensor([40, 60, 0, 250, 100], dtype=torch.int32, device=DEV)
    rep = torch.tensor([1.3, 1.0, 1.0, 2.0, 1.1], device=DEV)
    freq = torch.tensor([0.0, 0.5, 0.0, 0.0, 0.2], device=DEV)
    pres = torch.tensor([0.0, 0.0, 0.0, 0.7, 0.3], device=DEV)
    ref = S.apply_penalties_ref(logits.clone(), hist, npr, rep, freq, pres)
    got = S.apply_penalties(logits.clone(), hist, npr, rep, freq, pres)
    _close(got, ref, 1e-2, 1e-2)
    assert torch.equal(got[2], logits[2])
