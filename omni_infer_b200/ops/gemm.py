"""Dense and grouped GEMMs (bf16 and block-scaled e4m3) with fused SwiGLU / quant epilogues.

CUDA tensors run ``csrc/kernels/gemm_sm100.cu`` (tcgen05 + TMEM, weights as the UMMA M
dimension); CPU tensors run the fp32 reference below, which is also the oracle of the tests.
Plays the role of the reference's ``npu_quant_matmul`` / ``npu_grouped_matmul`` /
``npu_dequant_swiglu_quant`` call sites (omni/models/common/layers/moe/fused_moe/fused_moe.py:541-575).
"""
from __future__ import annotations

import torch

from . import _native as nat

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
_EPI = {"store": 0, "swiglu": 1, "swiglu_quant": 2}


def quant_fp8_block_ref(x: torch.Tensor, block: int = 128, ld: int | None = None):
    """Per-(row, 128-column block) e4m3 quantisation.  Returns (x_q [T,K], scale_t [K/128, ld])."""
    T, K = x.shape
    nb = (K + block - 1) // block
    xf = x.float()
    pad = nb * block - K
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    xb = xf.view(T, nb, block)
    amax = xb.abs().amax(dim=-1).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (xb / scale.unsqueeze(-1)).view(T, nb * block)[:, :K].to(FP8)
    ld = T if ld is None else ld
    st = torch.zeros(nb, ld, dtype=torch.float32, device=x.device)
    st[:, :T] = scale.t()
    return q, st


def quant_weight_fp8_block_ref(w: torch.Tensor, block: int = 128):
    """128x128 block e4m3 quantisation of a weight [..., N, K] -> (w_q, scale [..., N/128, K/128])."""
    *lead, N, K = w.shape
    nb_n, nb_k = (N + block - 1) // block, (K + block - 1) // block
    wf = w.float()
    wf = torch.nn.functional.pad(wf, (0, nb_k * block - K, 0, nb_n * block - N))
    wb = wf.view(*lead, nb_n, block, nb_k, block)
    amax = wb.abs().amax(dim=(-3, -1)).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (wb / scale[..., :, None, :, None]).view(*lead, nb_n * block, nb_k * block)[..., :N, :K].to(FP8)
    return q.contiguous(), scale.contiguous()


def dequant_weight_ref(wq: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    *lead, N, K = wq.shape
    s = scale.repeat_interleave(block, dim=-2)[..., :N, :].repeat_interleave(block, dim=-1)[..., :K]
    return wq.float() * s


def dequant_act_ref(xq: torch.Tensor, scale_t: torch.Tensor, block: int = 128) -> torch.Tensor:
    T, K = xq.shape
    s = scale_t[:, :T].t().repeat_interleave(block, dim=-1)[:, :K]
    return xq.float() * s


def gemm_ref(x, w, *, w_scale=None, x_scale=None, seg_start=None, seg_len=None, epi="store",
             row_scale=None, out_dtype=torch.bfloat16, out_scale_ld=None):
    """fp32 reference of :func:`gemm` with identical argument conventions."""
    if w.dim() == 2:
        w = w.unsqueeze(0)
        if w_scale is not None:
            w_scale = w_scale.unsqueeze(0)
    G = w.shape[0]
    T = x.shape[0]
    xf = dequant_act_ref(x, x_scale) if x.dtype == FP8 else x.float()
    wf = dequant_weight_ref(w, w_scale) if w.dtype == FP8 else w.float()
    n_w = w.shape[1]
    n_out = n_w if epi == "store" else n_w // 2
    y = torch.zeros(T, n_out, dtype=torch.float32, device=x.device)
    if seg_len is None:
        starts, lens = [0], [T]
    else:
        starts, lens = seg_start.tolist(), seg_len.tolist()
    for g in range(G):
        s, l = starts[g], lens[g]
        if l == 0:
            continue
        acc = xf[s:s + l] @ wf[g].t()
        if epi != "store":
            acc = torch.nn.functional.silu(acc[:, :n_out]) * acc[:, n_out:]
        y[s:s + l] = acc
    if row_scale is not None:
        y = y * row_scale.float().unsqueeze(-1)
    if epi == "swiglu_quant":
        return quant_fp8_block_ref(y, ld=out_scale_ld if out_scale_ld else T)
    return y.to(out_dtype)


class TmCollective(nat.ctypes.Structure):
    """Collective side of a token-major GEMM call (mirrors OmniTmCollective in gemm_tokmajor_sm100.cu)."""
    _fields_ = [("rs_world", nat.ctypes.c_int), ("rs_rank", nat.ctypes.c_int), ("rs_rows_per_rank", nat.ctypes.c_int),
                ("pad0", nat.ctypes.c_int), ("rs_out", nat.ctypes.c_void_p * 8), ("rs_flag", nat.ctypes.c_void_p * 8),
                ("rs_done", nat.ctypes.c_void_p), ("rs_epoch", nat.ctypes.c_void_p),
                ("ag_world", nat.ctypes.c_int), ("ag_rank", nat.ctypes.c_int), ("ag_rows_per_rank", nat.ctypes.c_int),
                ("pad1", nat.ctypes.c_int), ("ag_flag", nat.ctypes.c_void_p), ("ag_epoch", nat.ctypes.c_void_p),
                ("ag_wait_ns", nat.ctypes.c_ulonglong)]


def _tm2(kind, e, w, x, out, G, n_out, K, T, seg_start, seg_len, w_scale, x_scale, out_f32, out_scale, row_scale,
         x_group_col=0, out_group_col=0, out_ld=None, x_ld=None, coll=None):
    rc = nat.lib().omni_gemm_tm2(
        nat.c_int(kind), nat.c_int(e), nat.ptr(w), nat.ptr(x), nat.ptr(out), nat.c_int(G), nat.c_int(n_out), nat.c_int(K),
        nat.c_int(T), nat.c_int(T), nat.ptr(seg_start), nat.ptr(seg_len), nat.ptr(w_scale), nat.ptr(x_scale),
        nat.c_int(x_scale.shape[1] if x_scale is not None else 0),
        nat.c_int(out_ld if out_ld is not None else out.stride(0)), nat.c_int(out_f32), nat.ptr(out_scale),
        nat.c_int(out_scale.shape[1] if out_scale is not None else 0), nat.ptr(row_scale),
        nat.c_int(x_group_col), nat.c_int(out_group_col), nat.c_int(x_ld if x_ld is not None else x.stride(0)),
        nat.ctypes.byref(coll) if coll is not None else None,
        nat.ptr(nat.status_buffer(x.device)), nat.stream())
    nat.check_rc(rc, "omni_gemm_tm2")


def gemm(x, w, *, w_scale=None, x_scale=None, seg_start=None, seg_len=None, epi="store",
         row_scale=None, out_dtype=None, out=None, out_scale=None, bn=0, t_hint=0):
    """``out[t] = epi(x[t] @ w[g(t)].T)``.

    x: [T, K] bf16 or e4m3 (then ``x_scale`` is [K/128, ld] fp32, K-block major).
    w: [N, K] or [G, N, K]; e4m3 weights carry ``w_scale`` [G, N/128, K/128].
    seg_start/seg_len: int32 [G] row segments per group (grouped GEMM).
    epi: "store" | "swiglu" (w holds gate rows then up rows) | "swiglu_quant" (returns (q, scale_t)).
    """
    if out_dtype is None:
        out_dtype = torch.bfloat16 if (x.dtype == FP8 or x.is_cuda) else x.dtype
    if not x.is_cuda:
        return gemm_ref(x, w, w_scale=w_scale, x_scale=x_scale, seg_start=seg_start, seg_len=seg_len,
                        epi=epi, row_scale=row_scale, out_dtype=out_dtype)
    L = nat.lib()
    if w.dim() == 2:
        w = w.unsqueeze(0)
    G, n_w, K = w.shape
    T = x.shape[0]
    assert x.shape[1] == K and x.stride(1) == 1 and w.is_contiguous()
    kind = 1 if x.dtype == FP8 else 0
    assert (w.dtype == FP8) == (kind == 1), "x and w must both be bf16 or both e4m3"
    if kind == 0:
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    e = _EPI[epi]
    n_out = n_w if e == 0 else n_w // 2
    if e == 1 and n_out % 128 != 0:
        # the fused SwiGLU epilogue pairs 128-row gate and up blocks; odd widths (e.g. 10944) take the plain GEMM
        # and a separate activation kernel
        from .basic import silu_mul
        both = gemm(x, w, w_scale=w_scale, x_scale=x_scale, seg_start=seg_start, seg_len=seg_len, epi="store",
                    row_scale=row_scale, out_dtype=torch.bfloat16, bn=bn, t_hint=t_hint)
        return silu_mul(both)
    if e == 2:
        if out is None:
            out = torch.empty(T, n_out, dtype=FP8, device=x.device)
        if out_scale is None:
            out_scale = torch.empty(n_out // 128, max(4, (T + 3) // 4 * 4), dtype=torch.float32, device=x.device)
        out_f32 = 0
    else:
        if out is None:
            out = torch.empty(T, n_out, dtype=out_dtype if e == 0 else torch.bfloat16, device=x.device)
        out_f32 = 1 if out.dtype == torch.float32 else 0
    tm_ok = n_out % 8 == 0 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
    # fp8: always token-major (one scale multiplier per thread and K block).  bf16: token-major from 64 rows per
    # group on (vector stores, N = 256 tiles); below that, and for the split-K fp32 router GEMM, tokens stay on N.
    rows_hint = t_hint if (seg_len is not None and t_hint > 0) else T
    if tm_ok and e != 2 and kind == 0 and rows_hint >= 64 and not out_f32 and bn == 0:
        _tm2(0, e, w, x, out, G, n_out, K, T, seg_start, seg_len, None, None, 0, None, row_scale)
        return out
    if tm_ok and kind == 1:
        _tm2(1, e, w, x, out, G, n_out, K, T, seg_start, seg_len, w_scale, x_scale, out_f32, out_scale, row_scale)
        if e == 2:
            return out, out_scale
        return out
    rc = L.omni_gemm(
        nat.c_int(kind), nat.c_int(e), nat.ptr(w), nat.ptr(x), nat.ptr(out), nat.c_int(G), nat.c_int(n_out),
        nat.c_int(K), nat.c_int(T), nat.c_int(T), nat.ptr(seg_start), nat.ptr(seg_len), nat.ptr(w_scale),
        nat.ptr(x_scale), nat.c_int(x_scale.shape[1] if x_scale is not None else 0),
        nat.c_int(out.stride(0)), nat.c_int(out_f32), nat.ptr(out_scale),
        nat.c_int(out_scale.shape[1] if out_scale is not None else 0), nat.ptr(row_scale),
        nat.c_int(0), nat.c_int(0), nat.c_int(x.stride(0)), nat.c_int(bn), nat.c_int(t_hint), nat.ptr(nat.status_buffer(x.device)), nat.stream())
    nat.check_rc(rc, "omni_gemm")
    if e == 2:
        return out, out_scale
    return out


def bmm_heads_ref(x, w):
    """x [T, H, K], w [H, N, K] -> [T, H, N] (fp32 accumulate)."""
    return torch.einsum("thk,hnk->thn", x.float(), w.float()).to(x.dtype)


def bmm_heads(x, w, out=None, out_col_offset=0):
    """Per-head GEMM without transposes: ``out[t, h, :N] = x[t, h, :K] @ w[h].T``.

    ``x`` may be a strided view [T, H, K] of a wider [T, H, Dx] buffer (last dim contiguous) and ``out``
    a wider [T, H, Do] buffer: heads are addressed as column offsets of one 2-D tensor map, so the
    absorbed MLA projections (q_nope @ W_UK, o_latent @ W_UV) read and write the attention layouts
    directly (omni/models/common/layers/attention/deepseek_mla.py:209-235, 440-560)."""
    T, H, K = x.shape
    N = w.shape[1]
    if not x.is_cuda:
        y = bmm_heads_ref(x, w)
        if out is None:
            return y
        out[:, :, out_col_offset:out_col_offset + N] = y
        return out
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()
    assert x.stride(2) == 1 and x.stride(0) == H * x.stride(1), "x must be a [T, H, Dx] buffer view"
    if out is None:
        out = torch.empty(T, H, N, dtype=x.dtype, device=x.device)
    assert out.stride(2) == 1 and out.stride(0) == H * out.stride(1)
    base_out = out[:, :, out_col_offset:] if out_col_offset else out
    if (T >= 64 and N % 8 == 0 and out.stride(0) % 8 == 0 and out.stride(1) % 8 == 0 and base_out.data_ptr() % 16 == 0):
        _tm2(0, 0, w, x, base_out, H, N, K, T, None, None, None, None, 0, None, None,
             x_group_col=x.stride(1), out_group_col=out.stride(1), out_ld=out.stride(0), x_ld=x.stride(0))
        return out
    rc = nat.lib().omni_gemm(
        nat.c_int(0), nat.c_int(0), nat.ptr(w), nat.ptr(x), nat.ptr(base_out), nat.c_int(H), nat.c_int(N), nat.c_int(K),
        nat.c_int(T), nat.c_int(T), nat.ptr(None), nat.ptr(None), nat.ptr(None), nat.ptr(None), nat.c_int(0),
        nat.c_int(out.stride(0)), nat.c_int(0), nat.ptr(None), nat.c_int(0), nat.ptr(None),
        nat.c_int(x.stride(1)), nat.c_int(out.stride(1)), nat.c_int(x.stride(0)), nat.c_int(0), nat.c_int(T),
        nat.ptr(nat.status_buffer(x.device)), nat.stream())
    nat.check_rc(rc, "omni_gemm(bmm_heads)")
    return out
