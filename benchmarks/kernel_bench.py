#!/usr/bin/env python
"""Stand-alone timing of single kernels on one GPU (CUDA events, warm-up, L2-sized inputs), used for the
roofline notes under profiles/ and as the small workloads for ncu captures.

    python benchmarks/kernel_bench.py mla_decode --bq 64 --ctx 2048
    python benchmarks/kernel_bench.py gemm --kind fp8 --t 512 --n 7168 --k 16384
    python benchmarks/kernel_bench.py grouped --kind fp8 --experts 32 --tokens-per-expert 128 --n 4096 --k 7168 --epi swiglu_quant
"""
import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from omni_infer_b200 import ops  # noqa: E402
from omni_infer_b200.ops import attention as A  # noqa: E402
from omni_infer_b200.ops import _native as nat  # noqa: E402

PEAKS = {"hbm_gbs": 6533.2, "bf16_tflops": 1657.8}
try:
    PEAKS.update(json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json"))))
except Exception:  # noqa: BLE001
    pass


def timeit(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(iters):
        flush.zero_()                     # evict L2 between timed iterations
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    nat.check_status()
    ts.sort()
    return ts[len(ts) // 2]


def report(name, us, bytes_, flops, extra=None):
    out = {"kernel": name, "us": round(us, 1), "GB/s": round(bytes_ / us / 1e3, 1), "TFLOP/s": round(flops / us / 1e6, 1),
           "frac_hbm_of_measured": round(bytes_ / us / 1e3 / PEAKS["hbm_gbs"], 3),
           "frac_bf16_peak_of_measured": round(flops / us / 1e6 / PEAKS["bf16_tflops"], 3)}
    if extra:
        out.update(extra)
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["mla_decode", "gemm", "grouped", "fmha", "bmm"])
    ap.add_argument("--bq", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--kind", default="fp8")
    ap.add_argument("--t", type=int, default=512)
    ap.add_argument("--n", type=int, default=7168)
    ap.add_argument("--k", type=int, default=16384)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--tokens-per-expert", type=int, default=128)
    ap.add_argument("--epi", default="store")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    dev = "cuda"
    torch.manual_seed(0)
    if a.what == "mla_decode":
        bs = 128
        nb = a.bq * ((a.ctx + bs - 1) // bs) + 1
        cache = (torch.randn(nb, bs, 576, device=dev) * 0.5).bfloat16()
        bt = (torch.arange(nb - 1, device=dev, dtype=torch.int32) + 1).view(a.bq, -1).contiguous()
        q = (torch.randn(a.bq, a.heads, 576, device=dev) * 0.5).bfloat16()
        sl = torch.full((a.bq,), a.ctx, dtype=torch.int32, device=dev)
        us = timeit(lambda: A.mla_decode(q, cache, bt, sl, 1 / math.sqrt(192), num_splits=1), a.iters)
        report("mla_decode", us, a.bq * a.ctx * 1152, a.bq * a.ctx * a.heads * 2 * (576 + 512), {"bq": a.bq, "ctx": a.ctx, "heads": a.heads})
    elif a.what == "gemm":
        x = torch.randn(a.t, a.k, device=dev)
        w = torch.randn(a.n, a.k, device=dev) * 0.05
        if a.kind == "fp8":
            xq, xs = ops.quant_fp8_block(x.bfloat16())
            wq, ws = ops.quant_weight_fp8_block_ref(w)
            fn = lambda: ops.gemm(xq, wq, w_scale=ws, x_scale=xs)  # noqa: E731
            wb = a.n * a.k
        else:
            xb, wb_ = x.bfloat16(), w.bfloat16()
            fn = lambda: ops.gemm(xb, wb_)  # noqa: E731
            wb = a.n * a.k * 2
        us = timeit(fn, a.iters)
        report(f"gemm_{a.kind}", us, wb + a.t * a.k * (1 if a.kind == "fp8" else 2) + a.t * a.n * 2, 2.0 * a.t * a.n * a.k,
               {"T": a.t, "N": a.n, "K": a.k})
    elif a.what == "grouped":
        E, tpe = a.experts, a.tokens_per_expert
        rows = E * ((tpe + 15) // 16 * 16)
        x = torch.randn(rows, a.k, device=dev).bfloat16()
        nw = a.n * (1 if a.epi == "store" else 2)
        ss = torch.arange(E, device=dev, dtype=torch.int32) * ((tpe + 15) // 16 * 16)
        sl = torch.full((E,), tpe, dtype=torch.int32, device=dev)
        if a.kind == "fp8":
            xq, xs = ops.quant_fp8_block(x, ld=rows)
            wq = torch.empty(E, nw, a.k, dtype=ops.FP8, device=dev)
            ws = torch.empty(E, nw // 128, (a.k + 127) // 128, dtype=torch.float32, device=dev)
            for e in range(E):
                q_, s_ = ops.quant_weight_fp8_block_ref(torch.randn(nw, a.k, device=dev) * 0.05)
                wq[e], ws[e] = q_, s_
            fn = lambda: ops.gemm(xq, wq, w_scale=ws, x_scale=xs, seg_start=ss, seg_len=sl, epi=a.epi, t_hint=tpe)  # noqa: E731
            wbytes = E * nw * a.k
        else:
            wq = (torch.randn(E, nw, a.k, device=dev) * 0.05).bfloat16()
            fn = lambda: ops.gemm(x, wq, seg_start=ss, seg_len=sl, epi=a.epi, t_hint=tpe)  # noqa: E731
            wbytes = E * nw * a.k * 2
        us = timeit(fn, a.iters)
        report(f"grouped_{a.kind}_{a.epi}", us, wbytes, 2.0 * E * tpe * nw * a.k, {"E": E, "tokens_per_expert": tpe, "N": a.n, "K": a.k})
    elif a.what == "bmm":
        # per-head GEMM of the absorbed MLA projections: q_nope [T, H, 192 (128 used)] @ W_UK[h] -> [T, H, 576 (512 used)]
        H = a.heads
        q = (torch.randn(a.t, H, 192, device=dev) * 0.5).bfloat16()
        w = (torch.randn(H, a.n, a.k, device=dev) * 0.05).bfloat16()
        out = torch.empty(a.t, H, 576, dtype=torch.bfloat16, device=dev)
        us = timeit(lambda: ops.bmm_heads(q[:, :, :a.k], w, out=out), a.iters)
        report("bmm_heads_bf16", us, (a.t * H * a.k + H * a.n * a.k + a.t * H * a.n) * 2, 2.0 * a.t * H * a.n * a.k,
               {"T": a.t, "H": H, "N": a.n, "K": a.k})
    elif a.what == "fmha":
        H, L = 16, a.ctx
        q = (torch.randn(L, H, 192, device=dev) * 0.5).bfloat16()
        kv = (torch.randn(L, H * 256, device=dev) * 0.5).bfloat16()
        lat = (torch.randn(L, 576, device=dev) * 0.5).bfloat16()
        cu = torch.tensor([0, L], dtype=torch.int32, device=dev)
        us = timeit(lambda: A.mla_prefill(q, kv, lat, H, 128, 64, 128, cu, cu, 1 / math.sqrt(192), L, L), a.iters)
        report("fmha_mla_prefill", us, L * H * (192 + 256 + 128) * 2, H * L * L / 2 * 2 * (192 + 128), {"L": L, "heads": H})


if __name__ == "__main__":
    main()
