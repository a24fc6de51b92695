"""Row-wise ops around attention: RMSNorm(+residual)(+fp8 quant), block quantisation, MLA latent
norm + RoPE + paged-cache write, GQA RoPE + cache write, SwiGLU, embedding gather.

CUDA tensors run ``csrc/kernels/norm_rope.cu`` / ``sampler_misc.cu``; CPU tensors run the fp32
references here (they are also the oracles of the GPU tests).
"""
from __future__ import annotations

import torch

from . import _native as nat
from .gemm import FP8, quant_fp8_block_ref


# ----------------------------------------------------------------------------- RMSNorm
def rmsnorm_ref(x, weight, eps, residual=None, quant=False):
    if residual is not None:
        h = (x.float() + residual.float()).to(x.dtype)
        residual.copy_(h)
    else:
        h = x
    hf = h.float()
    y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)
    if quant:
        q, s = quant_fp8_block_ref(y, ld=max(4, (y.shape[0] + 3) // 4 * 4))
        return y, q, s
    return y


def rmsnorm(x, weight, eps=1e-6, residual=None, quant=False, need_bf16=True):
    """y = rmsnorm(x + residual) * weight.  ``residual`` is updated in place to ``x + residual``.
    With ``quant`` also returns (y_q e4m3, scale_t [H/128, ld]) for a block-scaled GEMM that follows."""
    if not x.is_cuda:
        return rmsnorm_ref(x, weight, eps, residual, quant)
    T, H = x.shape
    assert x.stride(1) == 1 and x.dtype == torch.bfloat16
    out = torch.empty(T, H, dtype=x.dtype, device=x.device) if (need_bf16 or not quant) else None
    q = s = None
    ld = 0
    if quant:
        ld = max(4, (T + 3) // 4 * 4)
        q = torch.empty(T, H, dtype=FP8, device=x.device)
        s = torch.empty(H // 128, ld, dtype=torch.float32, device=x.device)
    rc = nat.lib().omni_rmsnorm(nat.ptr(x), nat.ptr(residual), nat.ptr(weight), nat.ptr(out), nat.ptr(q), nat.ptr(s),
                                nat.c_int(ld), nat.c_int(T), nat.c_int(H), nat.c_int(x.stride(0)),
                                nat.c_float(eps), nat.stream())
    nat.check_rc(rc, "omni_rmsnorm")
    if quant:
        return out, q, s
    return out


def quant_fp8_block(x, ld=None):
    """bf16 [T,K] -> (e4m3 [T,K], scale_t [K/128, ld]) with one scale per (row, 128 columns)."""
    T, K = x.shape
    ld = max(4, (T + 3) // 4 * 4) if ld is None else ld
    if not x.is_cuda:
        return quant_fp8_block_ref(x, ld=ld)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = torch.empty((K + 127) // 128, ld, dtype=torch.float32, device=x.device)
    rc = nat.lib().omni_quant_fp8_block(nat.ptr(x), nat.ptr(q), nat.ptr(s), nat.c_int(ld), nat.c_int(T), nat.c_int(K),
                                        nat.c_int(x.stride(0)), nat.ptr(None), nat.stream())
    nat.check_rc(rc, "omni_quant_fp8_block")
    return q, s


def silu_mul_ref(x):
    i = x.shape[-1] // 2
    return (torch.nn.functional.silu(x[..., :i].float()) * x[..., i:].float()).to(x.dtype)


def silu_mul(x):
    if not x.is_cuda:
        return silu_mul_ref(x)
    T, I2 = x.shape
    out = torch.empty(T, I2 // 2, dtype=x.dtype, device=x.device)
    rc = nat.lib().omni_silu_mul(nat.ptr(x.contiguous()), nat.ptr(out), nat.c_int(T), nat.c_int(I2 // 2), nat.stream())
    nat.check_rc(rc, "omni_silu_mul")
    return out


# ----------------------------------------------------------------------------- RoPE tables
def rope_cos_sin_table(rot_dim, max_pos, base=10000.0, scaling=None, device="cpu"):
    """[max_pos, rot_dim] fp32 = cos(rot_dim/2) | sin(rot_dim/2).  ``scaling`` may describe YaRN
    (keys factor, original_max_position_embeddings, beta_fast, beta_slow, mscale, mscale_all_dim):
    inverse frequencies are blended and cos/sin are multiplied by the YaRN attention factor
    (omni/models/common/layers/rotary_embedding.py:375-520); ``type`` linear, llama3 and dynamic are the other
    variants of that file (:312, :352)."""
    import math

    half = rot_dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float64) * 2 / rot_dim))
    mscale = 1.0
    if scaling and scaling.get("factor", 1.0) > 1.0 and scaling.get("type", scaling.get("rope_type", "yarn")) in ("yarn", "deepseek_yarn"):
        factor = float(scaling["factor"])
        orig = int(scaling.get("original_max_position_embeddings", 4096))
        beta_fast, beta_slow = scaling.get("beta_fast", 32), scaling.get("beta_slow", 1)

        def corr_dim(rot):
            return (rot_dim * math.log(orig / (rot * 2 * math.pi))) / (2 * math.log(base))

        low = max(math.floor(corr_dim(beta_fast)), 0)
        high = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(half, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        inv_mask = 1.0 - ramp
        inv_freq = inv_freq / factor * (1 - inv_mask) + inv_freq * inv_mask

        def ys(scale, ms):
            return 1.0 if scale <= 1 else 0.1 * ms * math.log(scale) + 1.0

        mscale = ys(factor, scaling.get("mscale", 1.0)) / ys(factor, scaling.get("mscale_all_dim", 0.0))
    elif scaling and scaling.get("type", scaling.get("rope_type")) == "linear":
        inv_freq = inv_freq / float(scaling["factor"])
    elif scaling and scaling.get("type", scaling.get("rope_type")) == "llama3":
        # Llama-3.1 extension (reference: rotary_embedding.py:352-373): wavelengths longer than the original context
        # divided by low_freq_factor are slowed down by `factor`, those shorter than it divided by high_freq_factor
        # are kept, the band between is interpolated
        factor = float(scaling.get("factor", 8.0))
        lo_f, hi_f = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        orig = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv_freq
        smooth = ((orig / wavelen - lo_f) / (hi_f - lo_f)).clamp(0, 1)
        inv_freq = torch.where(wavelen > orig / lo_f, inv_freq / factor,
                               torch.where(wavelen < orig / hi_f, inv_freq, (1 - smooth) * inv_freq / factor + smooth * inv_freq))
    elif scaling and scaling.get("type", scaling.get("rope_type")) == "dynamic":
        # dynamic NTK: the base grows with the table length beyond the original context
        factor = float(scaling.get("factor", 1.0))
        orig = int(scaling.get("original_max_position_embeddings", max_pos))
        if max_pos > orig:
            nb = base * ((factor * max_pos / orig) - (factor - 1)) ** (rot_dim / (rot_dim - 2))
            inv_freq = 1.0 / (nb ** (torch.arange(0, half, dtype=torch.float64) * 2 / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float64)
    ang = torch.outer(t, inv_freq)
    return torch.cat([ang.cos() * mscale, ang.sin() * mscale], dim=-1).float().to(device)


def rope_interleaved_ref(x, cos_sin, positions):
    """x [T, ..., D] rotated on interleaved pairs (x[2i], x[2i+1]) by angle pos * inv_freq[i]."""
    D = x.shape[-1]
    cs = cos_sin[positions]
    cos, sin = cs[:, : D // 2], cs[:, D // 2:]
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    xf = x.float()
    a, b = xf[..., 0::2], xf[..., 1::2]
    out = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
    return out.to(x.dtype)


def rope_neox_ref(x, cos_sin, positions):
    D = x.shape[-1]
    cs = cos_sin[positions]
    cos, sin = cs[:, : D // 2], cs[:, D // 2:]
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    xf = x.float()
    a, b = xf[..., : D // 2], xf[..., D // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


# ----------------------------------------------------------------------------- MLA latent write
def mla_kv_rope_cache_ref(latent, kv_weight, eps, cos_sin, positions, slots, cache, q=None, q_rope_off=0,
                          q_out=None, q_out_off=0):
    kvl = kv_weight.shape[0]
    rd = cos_sin.shape[1]
    ckv = rmsnorm_ref(latent[:, :kvl], kv_weight, eps)
    kpe = rope_interleaved_ref(latent[:, kvl:kvl + rd], cos_sin, positions)
    row = torch.cat([ckv, kpe], dim=-1)
    ok = slots >= 0
    if cache is not None:
        cache.view(-1, cache.shape[-1])[slots[ok], :kvl + rd] = row[ok].to(cache.dtype)
    if q is not None:
        rot = rope_interleaved_ref(q[..., q_rope_off:q_rope_off + rd], cos_sin, positions)
        if q_out is not None:
            q_out[..., q_out_off:q_out_off + rd] = rot
        else:
            q[..., q_rope_off:q_rope_off + rd] = rot
    return row


def mla_kv_rope_cache(latent, kv_weight, eps, cos_sin, positions, slots, cache, q=None, q_rope_off=0,
                      want_latent=False, q_out=None, q_out_off=0):
    """latent [T, >=576] -> normalised c_kv (512) | roped k_pe (64) written to ``cache`` rows ``slots``
    (slot < 0 skips the write); optionally rotates ``q[..., q_rope_off:q_rope_off+64]`` in place, or into
    ``q_out[..., q_out_off:q_out_off+64]`` when given (the absorbed-q buffer of the decode path).
    Returns the processed latent rows when ``want_latent`` (prefill needs them for the up-projection)."""
    if not latent.is_cuda:
        return mla_kv_rope_cache_ref(latent, kv_weight, eps, cos_sin, positions, slots, cache, q, q_rope_off,
                                     q_out, q_out_off)
    T = latent.shape[0]
    assert kv_weight.shape[0] == 512 and cos_sin.shape[1] == 64, "the sm_100a kernel is specialised for 512 + 64"
    out = torch.empty(T, 576, dtype=latent.dtype, device=latent.device) if want_latent else None
    heads = q.shape[1] if q is not None else 0
    qhd = q.shape[2] if q is not None else 0
    if q is not None:
        assert q.is_contiguous()
    cache2 = cache.view(-1, cache.shape[-1]) if cache is not None else None
    rc = nat.lib().omni_mla_kv_rope_cache(
        nat.ptr(latent), nat.c_int(latent.stride(0)), nat.ptr(kv_weight), nat.c_float(eps), nat.ptr(cos_sin),
        nat.ptr(positions), nat.ptr(slots), nat.ptr(cache2), nat.c_int(cache2.stride(0) if cache2 is not None else 0),
        nat.ptr(q), nat.c_int(heads), nat.c_int(qhd), nat.c_int(q_rope_off), nat.ptr(q_out),
        nat.c_int(q_out.shape[2] if q_out is not None else 0), nat.c_int(q_out_off), nat.ptr(out), nat.c_int(T),
        nat.stream())
    nat.check_rc(rc, "omni_mla_kv_rope_cache")
    return out


# ----------------------------------------------------------------------------- GQA rope + cache
def rope_qk_cache_ref(qkv, hq, hkv, D, cos_sin, positions, slots, k_cache, v_cache, q_norm_w=None, k_norm_w=None,
                      eps=1e-6):
    T = qkv.shape[0]
    v = qkv.view(T, hq + 2 * hkv, D)
    q, k, val = v[:, :hq], v[:, hq:hq + hkv], v[:, hq + hkv:]
    if q_norm_w is not None:
        q = rmsnorm_ref(q.reshape(-1, D), q_norm_w, eps).view(T, hq, D)
        k = rmsnorm_ref(k.reshape(-1, D), k_norm_w, eps).view(T, hkv, D)
    q = rope_neox_ref(q, cos_sin, positions)
    k = rope_neox_ref(k, cos_sin, positions)
    v[:, :hq] = q
    v[:, hq:hq + hkv] = k
    if slots is not None and k_cache is not None:
        ok = slots >= 0
        k_cache.view(-1, hkv, D)[slots[ok]] = k[ok]
        v_cache.view(-1, hkv, D)[slots[ok]] = val[ok]
    return qkv


def rope_qk_cache(qkv, hq, hkv, D, cos_sin, positions, slots, k_cache, v_cache, q_norm_w=None, k_norm_w=None,
                  eps=1e-6):
    """In place on ``qkv`` [T, (hq+2hkv)*D]: optional per-head RMSNorm on q/k, neox RoPE, and K/V rows
    scattered into the paged caches [slots, hkv, D]."""
    if not qkv.is_cuda:
        return rope_qk_cache_ref(qkv, hq, hkv, D, cos_sin, positions, slots, k_cache, v_cache, q_norm_w, k_norm_w, eps)
    assert qkv.is_contiguous()
    rc = nat.lib().omni_rope_qk_cache(nat.ptr(qkv), nat.c_int(hq), nat.c_int(hkv), nat.c_int(D), nat.ptr(q_norm_w),
                                      nat.ptr(k_norm_w), nat.c_float(eps), nat.ptr(cos_sin), nat.ptr(positions),
                                      nat.ptr(slots), nat.ptr(k_cache), nat.ptr(v_cache), nat.c_int(qkv.shape[0]),
                                      nat.stream())
    nat.check_rc(rc, "omni_rope_qk_cache")
    return qkv


# ----------------------------------------------------------------------------- embedding
def embedding(ids, table, vocab_start=0):
    """Vocab-parallel gather: rows outside [vocab_start, vocab_start + len(table)) come back zero."""
    vocab_end = vocab_start + table.shape[0]
    if not table.is_cuda:
        mine = (ids >= vocab_start) & (ids < vocab_end)
        out = table[(ids - vocab_start).clamp(0, table.shape[0] - 1)]
        return out * mine.unsqueeze(-1).to(out.dtype)
    T, H = ids.shape[0], table.shape[1]
    out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    rc = nat.lib().omni_embedding(nat.ptr(ids), nat.ptr(table), nat.c_int(T), nat.c_int(H), nat.c_int(vocab_start),
                                  nat.c_int(vocab_end), nat.ptr(out), nat.stream())
    nat.check_rc(rc, "omni_embedding")
    return out
