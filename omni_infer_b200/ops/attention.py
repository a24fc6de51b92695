"""Attention ops: MLA absorbed paged decode (``csrc/kernels/mla_decode.cu``), varlen causal prefill
and GQA paged decode (``csrc/kernels/fmha_sm100.cu``), with fp32 PyTorch references."""
from __future__ import annotations

import torch

from . import _native as nat


# ----------------------------------------------------------------------------- MLA decode
def mla_decode_ref(q, cache, block_table, seq_lens, scale, q_to_seq=None, kv_lora=512):
    """q [Bq, H, kv_lora+rope]; cache [blocks, block, >=kv_lora+rope]; returns [Bq, H, kv_lora] (latent space)."""
    Bq, H, D = q.shape
    bs = cache.shape[1]
    out = torch.zeros(Bq, H, kv_lora, dtype=torch.float32, device=q.device)
    flat = cache.reshape(-1, cache.shape[-1])[:, :D].float()
    for b in range(Bq):
        L = int(seq_lens[b])
        if L == 0:
            continue
        row = int(q_to_seq[b]) if q_to_seq is not None else b
        pos = torch.arange(L, device=q.device)
        slots = block_table[row, pos // bs].long() * bs + pos % bs
        kv = flat[slots]
        s = (q[b].float() @ kv.t()) * scale
        p = torch.softmax(s, dim=-1)
        out[b] = p @ kv[:, :kv_lora]
    return out.to(q.dtype)


_scratch = {}


def _mla_scratch(dev, n_o, n_l):
    key = (dev.index, "mla")
    buf = _scratch.get(key)
    if buf is None or buf[0].numel() < n_o or buf[1].numel() < n_l:
        buf = (torch.empty(max(n_o, 1 << 20), dtype=torch.float32, device=dev),
               torch.empty(max(n_l, 1 << 14), dtype=torch.float32, device=dev))
        _scratch[key] = buf
    return buf


def mla_decode(q, cache, block_table, seq_lens, scale, q_to_seq=None, num_splits=0, max_seq_len=None, kv_lora=512):
    """Absorbed MLA decode attention.  ``seq_lens[b]`` is the number of cache tokens q row b attends to
    (MTP rows of one request get consecutive lengths); ``q_to_seq`` maps q rows to block-table rows."""
    if not q.is_cuda:
        return mla_decode_ref(q, cache, block_table, seq_lens, scale, q_to_seq, kv_lora)
    Bq, H, D = q.shape
    assert D == 576 and kv_lora == 512, "the sm_100a kernel is specialised for kv_lora 512 + rope 64"
    assert D == 576 and q.is_contiguous() and q.dtype == torch.bfloat16
    bs = cache.shape[1]
    cache2 = cache.view(-1, cache.shape[-1])
    if num_splits <= 0:
        # enough CTAs to fill the GPU: 2 (dim halves) x splits x Bq >= ~2 waves when rows are few
        num_splits = 1
        if max_seq_len is not None and Bq * 2 < 148:
            want = max(1, 296 // (Bq * 2))
            tiles = (max_seq_len + 31) // 32
            num_splits = max(1, min(want, tiles // 4 if tiles >= 4 else 1, 32))
    out = torch.empty(Bq, H, 512, dtype=q.dtype, device=q.device)
    o_part = lse = None
    if num_splits > 1:
        o_part, lse = _mla_scratch(q.device, Bq * num_splits * H * 512, Bq * num_splits * H)
    rc = nat.lib().omni_mla_decode(
        nat.ptr(q), nat.ptr(cache2), nat.c_int(cache2.stride(0)), nat.ctypes.c_longlong(cache2.shape[0]),
        nat.ptr(block_table), nat.c_int(block_table.stride(0)), nat.ptr(seq_lens), nat.ptr(q_to_seq), nat.c_int(Bq),
        nat.c_int(H), nat.c_int(bs), nat.c_float(scale), nat.c_int(num_splits), nat.ptr(out), nat.ptr(o_part),
        nat.ptr(lse), nat.ptr(nat.status_buffer(q.device)), nat.stream())
    nat.check_rc(rc, "omni_mla_decode")
    return out


# ----------------------------------------------------------------------------- varlen causal prefill
def attn_prefill_ref(q, k, v, cu_q, cu_k, scale, causal=True):
    """q [Tq, Hq, Dqk], k [Tk, Hkv, Dqk], v [Tk, Hkv, Dv]; ragged by cu_q / cu_k; causal aligned to the
    end of the key range (query i of a request sees keys up to len_k - len_q + i)."""
    Tq, Hq, _ = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    out = torch.zeros(Tq, Hq, v.shape[-1], dtype=torch.float32, device=q.device)
    nb = cu_q.numel() - 1
    for b in range(nb):
        q0, q1 = int(cu_q[b]), int(cu_q[b + 1])
        k0, k1 = int(cu_k[b]), int(cu_k[b + 1])
        if q1 == q0:
            continue
        qq = q[q0:q1].float().transpose(0, 1)                      # [Hq, Lq, D]
        kk = k[k0:k1].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vv = v[k0:k1].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.matmul(qq, kk.transpose(1, 2)) * scale
        if causal:
            Lq, Lk = q1 - q0, k1 - k0
            i = torch.arange(Lq, device=q.device)[:, None]
            j = torch.arange(Lk, device=q.device)[None, :]
            s = s.masked_fill(j > i + (Lk - Lq), float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.matmul(p, vv).transpose(0, 1)
    return out.to(q.dtype)


def gqa_decode_ref(q, k_cache, v_cache, block_table, seq_lens, scale):
    """q [B, Hq, D]; caches [blocks, block, Hkv, D]."""
    B, Hq, D = q.shape
    bs, Hkv = k_cache.shape[1], k_cache.shape[2]
    rep = Hq // Hkv
    out = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    kf = k_cache.reshape(-1, Hkv, D).float()
    vf = v_cache.reshape(-1, Hkv, D).float()
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        pos = torch.arange(L, device=q.device)
        slots = block_table[b, pos // bs].long() * bs + pos % bs
        kk = kf[slots].transpose(0, 1).repeat_interleave(rep, dim=0)   # [Hq, L, D]
        vv = vf[slots].transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.einsum("hd,hld->hl", q[b].float(), kk) * scale
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hl,hld->hd", p, vv)
    return out.to(q.dtype)


def mla_prefill_ref(q, kv, lat, H, nope, rope, vd, cu_q, cu_k, scale):
    """Non-absorbed MLA prefill: q [Tq, H, nope+rope] (rope already applied), kv [Tk, H*(nope+vd)] = per head
    k_nope | v, lat [Tk, kv_lora+rope] whose last ``rope`` columns are the shared roped k_pe."""
    Tk = kv.shape[0]
    kvh = kv.view(Tk, H, nope + vd)
    k_pe = lat[:, -rope:].unsqueeze(1).expand(Tk, H, rope)
    k = torch.cat([kvh[:, :, :nope], k_pe.to(kv.dtype)], dim=-1)
    v = kvh[:, :, nope:]
    return attn_prefill_ref(q, k, v, cu_q, cu_k, scale, causal=True)


def mla_prefill(q, kv, lat, H, nope, rope, vd, cu_q, cu_k, scale, max_q, max_k):
    if not q.is_cuda:
        return mla_prefill_ref(q, kv, lat, H, nope, rope, vd, cu_q, cu_k, scale)
    from .fmha import fmha_varlen
    kvl = lat.shape[1] - rope
    return fmha_varlen(q.view(q.shape[0], H * (nope + rope)), kv, kv, cu_q, cu_k, scale, Hq=H, Hkv=H,
                       q_head_stride=nope + rope, k_head_stride=nope + vd, v_head_stride=nope + vd, v_col0=nope,
                       d_k1=nope, k2=lat, k2_col0=kvl, d_k2=rope, d_v=vd, max_q=max_q, max_k=max_k, causal=True)


def gqa_prefill(q, k, v, cu_q, cu_k, scale, max_q, max_k):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] (views allowed), causal varlen."""
    if not q.is_cuda:
        return attn_prefill_ref(q, k, v, cu_q, cu_k, scale, causal=True)
    from .fmha import fmha_varlen
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    return fmha_varlen(q, k, v, cu_q, cu_k, scale, Hq=Hq, Hkv=Hkv, q_head_stride=q.stride(1), k_head_stride=k.stride(1),
                       v_head_stride=v.stride(1), v_col0=0, d_k1=D, k2=None, k2_col0=0, d_k2=0, d_v=D, max_q=max_q,
                       max_k=max_k, causal=True)


def gqa_decode(q, k_cache, v_cache, block_table, seq_lens, scale, max_seq_len=None):
    if not q.is_cuda:
        return gqa_decode_ref(q, k_cache, v_cache, block_table, seq_lens, scale)
    from .fmha import gqa_paged_decode
    return gqa_paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale, max_seq_len)
