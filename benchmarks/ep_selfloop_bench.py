#!/usr/bin/env python
"""The expert-parallel dispatch / combine kernels with W ranks emulated on ONE GPU.

Every emulated rank gets its own region of one device buffer; ``peer[r]`` points at region r, exactly as the IPC-mapped
buffers do in a multi-GPU run.  The kernels of the W ranks are launched one after the other on one stream (all sends,
then all receives, ...), so a receive finds every flag already set and nothing ever waits for a kernel that has not run.
Peer stores therefore go to local HBM instead of over NVLink: the times say what the kernels cost on the device side
(quantisation, addressing, flags), and the script is the small single-GPU workload for ncu captures of these kernels.
The result is checked: with identity experts, combine(dispatch(x)) must equal sum_k w[t,k] * dequant(quant(x[t])).

    python benchmarks/ep_selfloop_bench.py --world 8 --tokens 512
"""
import argparse
import ctypes
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from omni_infer_b200 import ops  # noqa: E402
from omni_infer_b200.ops import FP8  # noqa: E402
from omni_infer_b200.ops import _native as nat  # noqa: E402
from omni_infer_b200.parallel.ep_fused import EpLayout, _align  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=512, help="token rows per emulated rank")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--experts-per-rank", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--prequant", action="store_true", help="hand already quantised rows to the dispatch (copy instead of quantise)")
    ap.add_argument("--payload", default="fp8", choices=["fp8", "bf16"], help="what the dispatched rows carry")
    a = ap.parse_args()
    W, T, H, k, S = a.world, a.tokens, a.hidden, a.topk, a.experts_per_rank
    dev = torch.device("cuda")
    L = nat.lib()
    cap = T * k
    pb = 2 if a.payload == "bf16" else 1
    lays = []
    off = 0
    for r in range(W):
        lay = EpLayout(world=W, rank=r, cap=cap, H=H, max_slots=T * k, payload=pb)
        off = 0
        for name, size in (("off_recv_x", W * cap * H * pb), ("off_recv_s", W * cap * (H // 128) * 4), ("off_recv_meta", W * cap * 16),
                           ("off_recv_cnt", 256), ("off_recv_flag", 256), ("off_comb", T * k * H * 2), ("off_comb_flag", 256),
                           ("off_ctrl", 256)):
            setattr(lay, name, off)
            off = _align(off + size)
        lays.append(lay)
    region = off
    buf = torch.zeros(W * region, dtype=torch.uint8, device=dev)
    peers = (ctypes.c_void_p * 16)(*([ctypes.c_void_p(buf.data_ptr() + r * region) for r in range(W)] + [None] * (16 - W)))
    g = torch.Generator(device="cuda").manual_seed(0)
    xs_ = [(torch.randn(T, H, device=dev, generator=g) * 0.5).bfloat16() for _ in range(W)]
    ids_ = [torch.stack([torch.randperm(W * S, device=dev, generator=g)[:k] for _ in range(T)]).int().contiguous() for _ in range(W)]
    ws_ = [torch.rand(T, k, device=dev, generator=g).float().contiguous() for _ in range(W)]
    pre = [ops.quant_fp8_block(x) for x in xs_] if (a.prequant and pb == 1) else None
    st = nat.ptr(nat.status_buffer(dev))
    n = W * cap
    capacity = (n + S * 15 + 15) // 16 * 16
    wait_ns = ctypes.c_ulonglong(2_000_000_000)
    names = ["dispatch_send", "dispatch_recv", "align", "scatter_q", "combine_send", "combine_reduce"]
    times = {m: [] for m in names}

    def timed(name, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        return name, e0, e1

    outs = None
    for it in range(a.iters + 2):
        evs = []
        for r in range(W):
            evs.append(timed("dispatch_send", lambda r=r: nat.check_rc(L.omni_ep_dispatch_send(
                nat.ptr(xs_[r]), nat.ptr(pre[r][0]) if pre else None, nat.ptr(pre[r][1]) if pre else None,
                nat.c_int(pre[r][1].shape[1] if pre else 0), nat.ptr(ids_[r]), nat.ptr(ws_[r]), nat.c_int(T), nat.c_int(k), nat.c_int(S),
                ctypes.byref(lays[r]), peers, st, nat.stream()), "send")))
        state = []
        for r in range(W):
            r_ids = torch.empty(n, dtype=torch.int32, device=dev); r_w = torch.empty(n, dtype=torch.float32, device=dev)
            r_slot = torch.empty(n, dtype=torch.int32, device=dev)
            evs.append(timed("dispatch_recv", lambda: nat.check_rc(L.omni_ep_dispatch_recv(
                ctypes.byref(lays[r]), peers, nat.ptr(r_ids), nat.ptr(r_w), nat.ptr(r_slot), nat.ptr(None), wait_ns, st,
                nat.stream()), "recv")))
            counts = torch.empty(S, dtype=torch.int32, device=dev); pos = torch.empty(n, dtype=torch.int32, device=dev)
            seg_start = torch.empty(S, dtype=torch.int32, device=dev); seg_len = torch.empty(S, dtype=torch.int32, device=dev)
            total = torch.empty(1, dtype=torch.int32, device=dev)
            evs.append(timed("align", lambda: nat.check_rc(L.omni_moe_align(
                nat.ptr(r_ids), nat.c_int(n), nat.c_int(0), nat.c_int(S), nat.c_int(16), nat.c_int(capacity), nat.ptr(counts),
                nat.ptr(pos), nat.ptr(seg_start), nat.ptr(seg_len), nat.ptr(total), st, nat.stream()), "align")))
            xq = torch.empty(capacity, H, dtype=FP8 if pb == 1 else torch.bfloat16, device=dev)
            xsc = torch.empty(H // 128, capacity, dtype=torch.float32, device=dev)
            row_w = torch.empty(capacity, dtype=torch.float32, device=dev)
            row_rank = torch.empty(capacity, dtype=torch.int32, device=dev); row_slot = torch.empty(capacity, dtype=torch.int32, device=dev)
            evs.append(timed("scatter_q", lambda: nat.check_rc(L.omni_ep_scatter_q(
                ctypes.byref(lays[r]), peers, nat.ptr(r_ids), nat.ptr(pos), nat.ptr(r_w), nat.ptr(r_slot), nat.ptr(seg_start),
                nat.ptr(seg_len), nat.ptr(xq), nat.ptr(xsc), nat.c_int(capacity), nat.ptr(row_w), nat.ptr(row_rank),
                nat.ptr(row_slot), nat.stream()), "scatter")))
            # identity experts: y = w * dequant(x); rows between segments are never sent back
            xf = ops.dequant_act_ref(xq, xsc) if pb == 1 else xq.float()
            y = (xf * row_w.unsqueeze(1)).to(torch.bfloat16)
            state.append((y, total, seg_start, seg_len, row_rank, row_slot))
        for r in range(W):
            y, total, seg_start, seg_len, row_rank, row_slot = state[r]
            evs.append(timed("combine_send", lambda: nat.check_rc(L.omni_ep_combine_send(
                nat.ptr(y), nat.ptr(total), nat.ptr(seg_start), nat.ptr(seg_len), nat.c_int(S), nat.ptr(row_rank),
                nat.ptr(row_slot), nat.c_int(capacity), ctypes.byref(lays[r]), peers, nat.stream()), "csend")))
        outs = []
        for r in range(W):
            out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
            evs.append(timed("combine_reduce", lambda: nat.check_rc(L.omni_ep_combine_reduce(
                ctypes.byref(lays[r]), peers, nat.ptr(ids_[r]), nat.c_int(T), nat.c_int(k), nat.ptr(None), nat.ptr(out), wait_ns,
                st, nat.stream()), "creduce")))
            outs.append(out)
        torch.cuda.synchronize()
        nat.check_status()
        if it >= 2:
            for name, e0, e1 in evs:
                times[name].append(e0.elapsed_time(e1) * 1e3)
    # check rank 0's result
    if pb == 1:
        xq0, xs0 = ops.quant_fp8_block(xs_[0])
        ref = ops.dequant_act_ref(xq0, xs0) * ws_[0].sum(1, keepdim=True)
    else:
        ref = xs_[0].float() * ws_[0].sum(1, keepdim=True)
    err = float((outs[0].float() - ref).abs().max() / ref.abs().max())
    med = {m: round(sorted(v)[len(v) // 2], 1) for m, v in times.items()}
    row_bytes = (H + (H // 128) * 4 if pb == 1 else 2 * H) + 16
    print(json.dumps({"emulated_world": W, "tokens_per_rank": T, "hidden": H, "top_k": k, "payload": a.payload, "prequantised_input": bool(pre), "us_per_launch_median": med,
                      "dispatch_payload_MB_per_rank": round(T * k * row_bytes / 1e6, 1),
                      "combine_payload_MB_per_rank": round(T * k * H * 2 / 1e6, 1), "rel_err_vs_reference": round(err, 4)}))
    assert err < 2e-2, err


if __name__ == "__main__":
    main()
