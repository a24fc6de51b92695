"""tcgen05 GEMM family vs the fp32 PyTorch reference of the same op."""
import pytest
import torch

import importlib

G = importlib.import_module("omni_infer_b200.ops.gemm")

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (7, 128, 128), (16, 256, 512), (33, 576, 2048), (64, 1536, 7168),
                                   (128, 384, 1408), (200, 512, 1024), (300, 256, 768)])
def test_dense_bf16(T, N, K):
    torch.manual_seed(0)
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    y = G.gemm(x, w)
    ref = G.gemm_ref(x, w)
    assert y.shape == ref.shape
    assert _rel_err(y, ref) < 1e-2


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
def test_dense_bf16_all_tiles(bn):
    torch.manual_seed(1)
    T, N, K = 260, 640, 1024
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    y = G.gemm(x, w, bn=bn, out_dtype=torch.float32)
    ref = G.gemm_ref(x, w, out_dtype=torch.float32)
    assert _rel_err(y, ref) < 5e-3


def test_dense_bf16_row_scale_and_f32():
    torch.manual_seed(2)
    T, N, K = 50, 256, 512
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    rs = torch.rand(T, device="cuda")
    y = G.gemm(x, w, row_scale=rs, out_dtype=torch.float32)
    ref = G.gemm_ref(x, w, row_scale=rs, out_dtype=torch.float32)
    assert _rel_err(y, ref) < 5e-3


def _segments(lens, align=16):
    starts, pos = [], 0
    for l in lens:
        starts.append(pos)
        pos += (l + align - 1) // align * align
    return starts, max(pos, 16)


@pytest.mark.parametrize("lens", [[5, 0, 70, 16], [64] * 8, [0, 0, 3, 0], [130, 1, 33, 257, 0, 12]])
def test_grouped_bf16_swiglu(lens):
    torch.manual_seed(3)
    Gn, inter, K = len(lens), 256, 512
    starts, rows = _segments(lens)
    x = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(Gn, 2 * inter, K, device="cuda") * 0.05).bfloat16()
    ss = torch.tensor(starts, dtype=torch.int32, device="cuda")
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    y = G.gemm(x, w, seg_start=ss, seg_len=sl, epi="swiglu", t_hint=max(lens))
    ref = G.gemm_ref(x, w, seg_start=ss, seg_len=sl, epi="swiglu")
    for s, l in zip(starts, lens):
        if l:
            assert _rel_err(y[s:s + l], ref[s:s + l]) < 2e-2


@pytest.mark.parametrize("T,N,K", [(4, 128, 128), (16, 256, 512), (64, 512, 2048), (100, 1536, 7168), (128, 384, 1024)])
def test_dense_fp8_block(T, N, K):
    torch.manual_seed(4)
    x = torch.randn(T, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    xq, xs = G.quant_fp8_block_ref(x, ld=(T + 3) // 4 * 4)
    wq, ws = G.quant_weight_fp8_block_ref(w)
    y = G.gemm(xq, wq, w_scale=ws, x_scale=xs, out_dtype=torch.float32)
    ref = G.gemm_ref(xq, wq, w_scale=ws, x_scale=xs, out_dtype=torch.float32)
    assert _rel_err(y, ref) < 2e-3          # same quantised inputs: only accumulation order differs
    assert _rel_err(y, x @ w.t()) < 8e-2    # and it tracks the unquantised product


@pytest.mark.parametrize("lens", [[5, 0, 40, 16], [64] * 8, [130, 1, 33, 0]])
@pytest.mark.parametrize("epi", ["swiglu", "swiglu_quant"])
def test_grouped_fp8_swiglu(lens, epi):
    torch.manual_seed(5)
    Gn, inter, K = len(lens), 256, 512
    starts, rows = _segments(lens)
    x = torch.randn(rows, K, device="cuda")
    w = torch.randn(Gn, 2 * inter, K, device="cuda") * 0.05
    xq, xs = G.quant_fp8_block_ref(x)
    wq, ws = G.quant_weight_fp8_block_ref(w)
    ss = torch.tensor(starts, dtype=torch.int32, device="cuda")
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ref = G.gemm_ref(xq, wq, w_scale=ws, x_scale=xs, seg_start=ss, seg_len=sl, epi="swiglu", out_dtype=torch.float32)
    if epi == "swiglu":
        y = G.gemm(xq, wq, w_scale=ws, x_scale=xs, seg_start=ss, seg_len=sl, epi="swiglu", t_hint=max(lens))
        for s, l in zip(starts, lens):
            if l:
                assert _rel_err(y[s:s + l], ref[s:s + l]) < 2e-2
    else:
        q, qs = G.gemm(xq, wq, w_scale=ws, x_scale=xs, seg_start=ss, seg_len=sl, epi="swiglu_quant", t_hint=max(lens))
        deq = G.dequant_act_ref(q, qs)
        for s, l in zip(starts, lens):
            if l:
                assert _rel_err(deq[s:s + l], ref[s:s + l]) < 6e-2
