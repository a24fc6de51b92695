"""Checkpoint loaders on CPU: Hugging Face tensor names into the fused engine layouts for (i) float checkpoints,
(ii) DeepSeek-V3-style e4m3 + ``weight_scale_inv`` 128x128, (iii) the int8 compressed-tensors layout (per-channel
``weight_scale`` / ``weight_offset``), which is re-quantised to block e4m3 at load; and a bound on what that
re-quantisation costs against an int8 x int8 oracle."""
import pytest
import torch

from omni_infer_b200.models import build_model
from omni_infer_b200.models.config import get_config
from omni_infer_b200.ops.gemm import FP8, dequant_weight_ref, gemm_ref, quant_fp8_block_ref, quant_weight_fp8_block_ref


def hf_tensors(model, cfg) -> dict:
    """The model's float weights under the checkpoint's names (fused projections split, experts one by one)."""
    out = {}
    for name, t in model.state_dict().items():
        t = t.float()
        if name.endswith("fused_qkv_a_proj.weight"):
            base = name[: -len("fused_qkv_a_proj.weight")]
            if cfg.q_lora_rank:
                out[base + "q_a_proj.weight"] = t[: cfg.q_lora_rank]
                out[base + "kv_a_proj_with_mqa.weight"] = t[cfg.q_lora_rank:]
            else:
                qd = cfg.num_attention_heads * cfg.qk_head_dim
                out[base + "q_proj.weight"], out[base + "kv_a_proj_with_mqa.weight"] = t[:qd], t[qd:]
        elif name.endswith("qkv_proj.weight") or name.endswith("qkv_proj.bias"):
            kind = name.rsplit(".", 1)[1]
            base = name[: -len("qkv_proj." + kind)]
            hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
            out[base + "q_proj." + kind] = t[: hq * d]
            out[base + "k_proj." + kind] = t[hq * d:(hq + hkv) * d]
            out[base + "v_proj." + kind] = t[(hq + hkv) * d:]
        elif name.endswith("gate_up_proj.weight"):
            base = name[: -len("gate_up_proj.weight")]
            half = t.shape[0] // 2
            out[base + "gate_proj.weight"], out[base + "up_proj.weight"] = t[:half], t[half:]
        elif name.endswith(".mlp.w13"):
            base = name[: -len("w13")]
            half = t.shape[1] // 2
            for e in range(t.shape[0]):
                out[f"{base}experts.{e}.gate_proj.weight"], out[f"{base}experts.{e}.up_proj.weight"] = t[e, :half], t[e, half:]
        elif name.endswith(".mlp.w2"):
            base = name[: -len("w2")]
            for e in range(t.shape[0]):
                out[f"{base}experts.{e}.down_proj.weight"] = t[e]
        else:
            out[name] = t
    return out


QUANTISED = ("_proj.weight", "kv_a_proj_with_mqa.weight")   # what a quantised checkpoint stores in 8 bits: the projections


def _is_quantised(name: str) -> bool:
    return name.endswith(QUANTISED) and "layers." in name


def _logits(model, cfg, ids):
    from omni_infer_b200.models.reference_fp32 import reference_for
    return reference_for(cfg, dict(model.state_dict())).logits(ids)


def _fresh(name, seed, **over):
    cfg = get_config(name, **over)
    m = build_model(cfg, device="cpu")
    g = torch.Generator().manual_seed(seed)
    for p in m.parameters():
        if p.dtype.is_floating_point and p.dtype != FP8:
            p.data.copy_(torch.randn(p.shape, generator=g) * (0.05 if p.dim() > 1 else 1.0) + (0.0 if p.dim() > 1 else 1.0))
    return cfg, m


@pytest.mark.parametrize("name,over", [("tiny-deepseek-v3", {}), ("tiny-qwen3-moe", {}),
                                       ("qwen2-small", {"dtype": "float32", "hidden_size": 256, "intermediate_size": 512,
                                                        "head_dim": 32, "vocab_size": 512})])
def test_float_checkpoint_round_trip(name, over):
    cfg, src = _fresh(name, 1, **over)
    _, dst = _fresh(name, 2, **over)
    ckpt = hf_tensors(src, cfg)
    # any order: the loader must not depend on the order of the shards
    items = list(ckpt.items())
    perm = torch.randperm(len(items), generator=torch.Generator().manual_seed(0)).tolist()
    loaded = dst.load_weights((items[i][0], items[i][1].clone()) for i in perm)
    a, b = src.state_dict(), dst.state_dict()
    assert set(a) == set(b)
    for k in a:
        assert torch.equal(a[k], b[k]), k
    assert {k for k in a} <= loaded | {k for k in a if k.endswith("_scale")}


def _fp8_cfg():
    # every projection width a multiple of 128, as the block scales want
    return dict(quantization="fp8_block", hidden_size=256, q_lora_rank=128, kv_lora_rank=128, qk_rope_head_dim=64,
                qk_nope_head_dim=64, v_head_dim=64, num_attention_heads=4, intermediate_size=512, moe_intermediate_size=128)


def test_fp8_block_checkpoint_loads_bit_exact():
    """e4m3 weights with ``weight_scale_inv`` go into the fused parameters unchanged (bytes and scales), also when
    two checkpoint tensors share one fused parameter and its scale rows."""
    over = _fp8_cfg()
    cfg_f, src = _fresh("tiny-deepseek-v3", 3, **{**over, "quantization": "none"})
    cfg_q, dst = _fresh("tiny-deepseek-v3", 4, **over)
    ckpt, want = {}, {}
    for k, t in hf_tensors(src, cfg_f).items():
        if _is_quantised(k):
            q, s = quant_weight_fp8_block_ref(t)
            ckpt[k], ckpt[k[: -len("weight")] + "weight_scale_inv"] = q, s
            want[k] = dequant_weight_ref(q, s)
        else:
            ckpt[k] = t
    dst.load_weights(list(ckpt.items()))
    sd = dst.state_dict()
    got = hf_tensors_dequant(dst, cfg_q)
    for k, w in want.items():
        assert torch.equal(got[k], w), k
    assert sd["model.layers.0.self_attn.q_b_proj.weight"].dtype == FP8
    # and the model runs: logits of the loaded model equal those of the oracle on the de-quantised weights
    ids = torch.randint(0, cfg_q.vocab_size, (12,), generator=torch.Generator().manual_seed(0)).tolist()
    assert torch.isfinite(_logits(dst, cfg_q, ids)).all()


def hf_tensors_dequant(model, cfg) -> dict:
    """hf_tensors of a quantised model, with every e4m3 parameter de-quantised first."""
    sd = model.state_dict()
    class _View:
        def state_dict(self_inner):
            out = {}
            for k, v in sd.items():
                if k.endswith("_scale"):
                    continue
                out[k] = dequant_weight_ref(v, sd[k + "_scale"]) if v.dtype == FP8 else v
            return out
    return hf_tensors(_View(), cfg)


@pytest.mark.parametrize("with_offset", [False, True])
def test_int8_compressed_tensors_checkpoint(with_offset):
    """int8 per-channel weights are de-quantised ((w - offset) * scale) and stored as block e4m3: every stored value
    is within e4m3 rounding of the checkpoint's value, and the model's logits stay close to the float model built
    from the same int8 values."""
    over = _fp8_cfg()
    cfg_f, src = _fresh("tiny-deepseek-v3", 5, **{**over, "quantization": "none"})
    cfg_q, dst = _fresh("tiny-deepseek-v3", 6, **over)
    g = torch.Generator().manual_seed(1)
    ckpt, meaning = {}, {}
    for k, t in hf_tensors(src, cfg_f).items():
        if not _is_quantised(k):
            ckpt[k] = meaning[k] = t
            continue
        off = torch.randint(-3, 4, (t.shape[0],), generator=g).float() if with_offset else torch.zeros(t.shape[0])
        scale = (t.abs().amax(1) / 120.0).clamp_min(1e-8)
        q = torch.round(t / scale[:, None] + off[:, None]).clamp(-128, 127).to(torch.int8)
        ckpt[k] = q
        ckpt[k[: -len("weight")] + "weight_scale"] = scale[:, None]
        if with_offset:
            ckpt[k[: -len("weight")] + "weight_offset"] = off[:, None]
        meaning[k] = (q.float() - off[:, None]) * scale[:, None]
    if with_offset:
        from omni_infer_b200.quantization.loader import WeightLoader
        wl = WeightLoader(dst, cfg_q)
        wl._expects_offset = True
        wl.load(list(ckpt.items()))
    else:
        dst.load_weights(list(ckpt.items()))
    got = hf_tensors_dequant(dst, cfg_q)
    for k, w in meaning.items():
        if not _is_quantised(k):
            assert torch.equal(got[k], w), k
            continue
        # e4m3 keeps 3 mantissa bits: half an ulp is 2^-4 of the value, plus the subnormal floor of the block
        tol = w.abs() * 2.0 ** -4 + w.abs().max() * 2.0 ** -9
        assert bool(((got[k] - w).abs() <= tol).all()), k
    # the float model that means the same as the checkpoint
    _, same = _fresh("tiny-deepseek-v3", 7, **{**over, "quantization": "none"})
    same.load_weights(list(meaning.items()))
    ids = torch.randint(0, cfg_q.vocab_size, (16,), generator=torch.Generator().manual_seed(2)).tolist()
    a, b = _logits(dst, cfg_q, ids), _logits(same, cfg_f, ids)
    cos = torch.nn.functional.cosine_similarity(a, b, dim=-1).min().item()
    assert cos > 0.99, cos      # e4m3 rounding of every projection weight, two layers deep


def test_int8_to_e4m3_drift_against_int8_oracle():
    """What the load-time conversion costs in a projection's output.  Oracle: the int8 x int8 GEMM the checkpoint was
    made for (activations quantised per token, weights per channel).  Ours: the same weights as block e4m3, the
    activations as e4m3 with one scale per 128 columns.  Both are measured against the exact product with the
    de-quantised int8 weights."""
    g = torch.Generator().manual_seed(0)
    T, K, N = 64, 2048, 1024
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    for outliers in (False, True):
        w = torch.randn(N, K, generator=g) * 0.02
        x = torch.randn(T, K, generator=g)
        if outliers:
            x[:, ::97] *= 20            # a few hot channels, as activations of real models have
        sw = w.abs().amax(1, keepdim=True) / 127
        wq = torch.round(w / sw).clamp(-127, 127)
        meant = wq * sw
        sx = x.abs().amax(1, keepdim=True) / 127
        xq = torch.round(x / sx).clamp(-127, 127)
        y_int8 = (xq @ wq.t()) * sx * sw.t()
        y_exact = x @ meant.t()
        w8, ws = quant_weight_fp8_block_ref(meant)
        x8, xs = quant_fp8_block_ref(x)
        y_fp8 = gemm_ref(x8, w8, w_scale=ws, x_scale=xs, out_dtype=torch.float32)
        e_int8, e_fp8, drift = rel(y_int8, y_exact), rel(y_fp8, y_exact), rel(y_fp8, y_int8)
        assert e_fp8 < 0.05 and drift < 0.065, (outliers, e_int8, e_fp8, drift)
        if outliers:
            assert e_fp8 < e_int8      # per-128-column scales absorb hot channels that a per-token scale cannot
        else:
            assert e_int8 < e_fp8      # on well-behaved inputs int8 is the finer grid: the cost of converting is real


@pytest.mark.parametrize("world,kv_heads,quant", [(2, 2, "none"), (4, 2, "none"), (2, 2, "fp8_block")])
def test_tensor_parallel_gqa_shards_load_this_ranks_heads(world, kv_heads, quant):
    """Checkpoint q/k/v/o tensors (and the qkv bias) into a model whose attention is sharded over ``world`` ranks: every
    rank holds its own query heads, the K/V heads it needs (replicated when there are fewer than ranks), and its
    columns of o_proj; for an e4m3 checkpoint bytes and scale blocks are taken over unchanged."""
    over = {"dtype": "float32", "hidden_size": 256, "intermediate_size": 512, "head_dim": 128, "vocab_size": 512,
            "num_attention_heads": 4, "num_key_value_heads": kv_heads}
    cfg, src = _fresh("qwen2-small", 1, **over)
    ckpt = hf_tensors(src, cfg)
    if quant == "fp8_block":
        for k in [k for k in ckpt if _is_quantised(k)]:
            q, s = quant_weight_fp8_block_ref(ckpt[k])
            ckpt[k], ckpt[k[: -len("weight")] + "weight_scale_inv"] = q, s
    hq, d = cfg.num_attention_heads, cfg.head_dim
    pre = "model.layers.1.self_attn."
    for rank in range(world):
        _, dst = _fresh("qwen2-small", 2 + rank, **over, attn_tp_size=world, attn_tp_rank=rank, quantization=quant)
        att = dst.model.layers[1].self_attn
        hql, hkvl, kv0 = att.Hq, att.Hkv, att.kv_head0
        assert (hql, hkvl, kv0) == (hq // world, max(1, kv_heads // world), rank * kv_heads // world)
        assert att.qkv_proj.weight.shape[0] == (hql + 2 * hkvl) * d and att.o_proj.weight.shape[1] == hql * d
        dst.load_weights([(k, v.clone()) for k, v in ckpt.items()])
        want_rows = {"q": slice(rank * hql * d, (rank + 1) * hql * d), "k": slice(kv0 * d, (kv0 + hkvl) * d),
                     "v": slice(kv0 * d, (kv0 + hkvl) * d)}
        got_rows = {"q": slice(0, hql * d), "k": slice(hql * d, (hql + hkvl) * d), "v": slice((hql + hkvl) * d, None)}
        w, b = att.qkv_proj.weight, att.qkv_proj.bias
        for kind in "qkv":
            full = ckpt[pre + kind + "_proj.weight"]
            if quant == "fp8_block":
                assert torch.equal(w[got_rows[kind]].view(torch.uint8), full[want_rows[kind]].view(torch.uint8))
                sc = ckpt[pre + kind + "_proj.weight_scale_inv"]
                g0 = got_rows[kind].start // 128
                n = (want_rows[kind].stop - want_rows[kind].start) // 128
                assert torch.equal(att.qkv_proj.weight_scale[g0:g0 + n], sc[want_rows[kind].start // 128:want_rows[kind].stop // 128])
            else:
                assert torch.equal(w[got_rows[kind]], full[want_rows[kind]])
            assert torch.equal(b[got_rows[kind]], ckpt[pre + kind + "_proj.bias"][want_rows[kind]])
        cols = slice(rank * hql * d, (rank + 1) * hql * d)
        if quant == "fp8_block":
            assert torch.equal(att.o_proj.weight.view(torch.uint8), ckpt[pre + "o_proj.weight"][:, cols].view(torch.uint8))
        else:
            assert torch.equal(att.o_proj.weight, ckpt[pre + "o_proj.weight"][:, cols])
        # the slice functions that the random initialisation uses pick the same rows of the merged tensor
        merged = torch.cat([ckpt[pre + k + "_proj.weight"].view(torch.uint8) if quant == "fp8_block" else ckpt[pre + k + "_proj.weight"]
                            for k in "qkv"], 0)
        assert torch.equal(att.qkv_proj.weight.tp_slice_fn(merged), w.view(torch.uint8) if quant == "fp8_block" else w)


@pytest.mark.parametrize("quant", ["none", "fp8_block"])
def test_shared_expert_ranks_load_pieces_of_the_shared_expert(quant, monkeypatch):
    """With dedicated shared-expert ranks the checkpoint's shared expert lands, piece by piece, in the first local slots
    of a shared rank (and nowhere on the others), routed experts only on the other ranks."""
    from omni_infer_b200.parallel import parallel_state as pst
    over = dict(_fp8_cfg(), quantization="none", n_shared_experts=2)
    cfg_f, src = _fresh("tiny-deepseek-v3", 5, **over)
    ckpt = hf_tensors(src, cfg_f)
    if quant == "fp8_block":
        for k in [k for k in ckpt if _is_quantised(k)]:
            q, s = quant_weight_fp8_block_ref(ckpt[k])
            ckpt[k], ckpt[k[: -len("weight")] + "weight_scale_inv"] = q, s
    I = cfg_f.moe_intermediate_size
    pre = "model.layers.1.mlp."

    def as_float(name):
        w = ckpt[name]
        return dequant_weight_ref(w, ckpt[name[: -len("weight")] + "weight_scale_inv"]) if w.dtype == FP8 else w

    def slot_float(moe, s):
        if quant == "fp8_block":
            return dequant_weight_ref(moe.w13[s], moe.w13_scale[s]), dequant_weight_ref(moe.w2[s], moe.w2_scale[s])
        return moe.w13[s].float(), moe.w2[s].float()

    st = pst.get_parallel_state()
    for rank in range(3):
        monkeypatch.setattr(st, "world_size", 3)
        monkeypatch.setattr(st, "rank", rank)
        _, dst = _fresh("tiny-deepseek-v3", 6, **{**over, "quantization": quant, "shared_expert_ranks": 1})
        monkeypatch.setattr(st, "world_size", 1)
        monkeypatch.setattr(st, "rank", 0)
        moe = dst.model.layers[1].mlp
        assert moe.shared_ranks == 1 and moe.slots_per_rank == 4 and moe.shared_experts is None
        with torch.no_grad():
            moe.w13.view(torch.uint8).zero_() if quant == "fp8_block" else moe.w13.zero_()
            moe.w2.view(torch.uint8).zero_() if quant == "fp8_block" else moe.w2.zero_()
        dst.load_weights([(k, v.clone()) for k, v in ckpt.items()])
        if rank == 0:
            g, u, d = (as_float(pre + f"shared_experts.{n}_proj.weight") for n in ("gate", "up", "down"))
            for j in range(2):
                w13, w2 = slot_float(moe, j)
                assert torch.equal(w13, torch.cat([g[j * I:(j + 1) * I], u[j * I:(j + 1) * I]], 0))
                assert torch.equal(w2, d[:, j * I:(j + 1) * I])
            for s in (2, 3):
                assert float(slot_float(moe, s)[0].abs().sum()) == 0.0
        else:
            for s in range(4):
                e = (rank - 1) * 4 + s
                w13, w2 = slot_float(moe, s)
                assert torch.equal(w13, torch.cat([as_float(pre + f"experts.{e}.gate_proj.weight"),
                                                   as_float(pre + f"experts.{e}.up_proj.weight")], 0))
                assert torch.equal(w2, as_float(pre + f"experts.{e}.down_proj.weight"))


def test_vocabulary_parallel_checkpoint_rows():
    """Each rank keeps its block of the embedding table and the LM head (the last block padded with zero rows)."""
    cfg, src = _fresh("tiny-deepseek-v3", 7, vocab_size=1000)
    ckpt = hf_tensors(src, cfg)
    per = (1000 + 2) // 3
    for rank in range(3):
        _, dst = _fresh("tiny-deepseek-v3", 8, vocab_size=1000, vocab_parallel_size=3, vocab_parallel_rank=rank)
        dst.load_weights([(k, v.clone()) for k, v in ckpt.items()])
        lo, hi = rank * per, min(1000, (rank + 1) * per)
        for got, name in ((dst.model.embed_tokens.weight, "model.embed_tokens.weight"), (dst.lm_head.weight, "lm_head.weight")):
            assert got.shape[0] == per
            assert torch.equal(got[: hi - lo], ckpt[name][lo:hi])
            assert float(got[hi - lo:].abs().sum()) == 0.0
