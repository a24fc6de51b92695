"""Host side of ``csrc/kernels/fmha_sm100.cu``: varlen causal prefill attention (tcgen05) and GQA paged
decode."""
from __future__ import annotations

import torch

from . import _native as nat

_scratch = {}


def _rows_ld_cols(t: torch.Tensor):
    """A 2-D or 3-D tensor whose trailing dims are contiguous per row -> (rows, row pitch, columns)."""
    rows = t.shape[0]
    ld = t.stride(0)
    cols = ld if t.dim() == 3 else t.shape[1]
    return rows, ld, cols


def fmha_varlen(q, k, v, cu_q, cu_k, scale, *, Hq, Hkv, q_head_stride, k_head_stride, v_head_stride, v_col0, d_k1,
                k2, k2_col0, d_k2, d_v, max_q, max_k, causal=True):
    """q: [Tq, ...] rows holding all heads (head h starts at column h*q_head_stride); k, v likewise with their own
    strides (they may be views into one buffer: only the data pointer, row pitch and column offsets matter);
    k2 [Tk, ...] optional extra key columns shared by all heads.  Returns [Tq, Hq, d_v] bf16."""
    assert q.dtype == torch.bfloat16 and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    Tq = q.shape[0]
    B = cu_q.numel() - 1
    out = torch.empty(Tq, Hq, d_v, dtype=q.dtype, device=q.device)
    q_rows, q_ld, _ = _rows_ld_cols(q)
    k_rows, k_ld, _ = _rows_ld_cols(k)
    _, v_ld, _ = _rows_ld_cols(v)
    # columns addressable from each base pointer (bounds of the tensor map)
    q_cols = (Hq - 1) * q_head_stride + d_k1 + d_k2
    k_cols = (Hkv - 1) * k_head_stride + d_k1
    v_cols = (Hkv - 1) * v_head_stride + v_col0 + d_v
    k2_ld = k2.stride(0) if k2 is not None else 0
    k2_cols = k2_col0 + d_k2 if k2 is not None else 0
    rc = nat.lib().omni_fmha_varlen(
        nat.ptr(q), nat.ctypes.c_longlong(q_rows), nat.c_int(q_ld), nat.c_int(q_cols),
        nat.ptr(k), nat.ctypes.c_longlong(k_rows), nat.c_int(k_ld), nat.c_int(k_cols),
        nat.ptr(k2), nat.c_int(k2_ld), nat.c_int(k2_cols), nat.ptr(v), nat.c_int(v_ld), nat.c_int(v_cols),
        nat.ptr(cu_q), nat.ptr(cu_k), nat.c_int(B), nat.c_int(max_q), nat.c_int(Hq), nat.c_int(Hkv),
        nat.c_int(q_head_stride), nat.c_int(k_head_stride), nat.c_int(v_head_stride), nat.c_int(v_col0),
        nat.c_int(k2_col0), nat.c_int(d_k1), nat.c_int(d_k2), nat.c_int(d_v), nat.c_float(scale),
        nat.c_int(1 if causal else 0), nat.ptr(out), nat.ptr(nat.status_buffer(q.device)), nat.stream())
    nat.check_rc(rc, "omni_fmha_varlen")
    return out


def gqa_paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale, max_seq_len=None, num_splits=0):
    """q [B, Hq, 128]; caches [blocks, block, Hkv, 128]; one query token per request."""
    B, Hq, D = q.shape
    Hkv, bs = k_cache.shape[2], k_cache.shape[1]
    assert q.is_contiguous() and q.dtype == torch.bfloat16
    if num_splits <= 0:
        # three CTAs fit an SM (shared memory and registers): aim for that many everywhere, but keep at least two
        # 32-key tiles per warp of a CTA so that the merge at the end stays small against the streaming part
        num_splits = 1
        ctas = B * Hkv
        if max_seq_len is not None and ctas < 444:
            tiles = (max_seq_len + 31) // 32
            num_splits = max(1, min((444 + ctas - 1) // ctas, tiles // 8, 32))
    out = torch.empty(B, Hq, D, dtype=q.dtype, device=q.device)
    o_part = lse = None
    if num_splits > 1:
        key = (q.device.index, "gqa")
        need_o, need_l = B * num_splits * Hq * D, B * num_splits * Hq
        buf = _scratch.get(key)
        if buf is None or buf[0].numel() < need_o:
            buf = (torch.empty(max(need_o, 1 << 20), dtype=torch.float32, device=q.device),
                   torch.empty(max(need_l, 1 << 14), dtype=torch.float32, device=q.device))
            _scratch[key] = buf
        o_part, lse = buf
    rc = nat.lib().omni_gqa_paged_decode(
        nat.ptr(q), nat.ptr(k_cache), nat.ptr(v_cache), nat.ptr(block_table), nat.c_int(block_table.stride(0)),
        nat.ptr(seq_lens), nat.c_int(B), nat.c_int(Hq), nat.c_int(Hkv), nat.c_int(D), nat.c_int(bs),
        nat.c_float(scale), nat.c_int(num_splits), nat.ptr(o_part), nat.ptr(lse), nat.ptr(out), nat.stream())
    nat.check_rc(rc, "omni_gqa_paged_decode")
    return out
