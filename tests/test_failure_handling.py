"""Failure handling on the GPU without faulting it: a cross-rank wait whose flag nobody sets runs into its (short)
limit, the kernel returns normally, the status word says where it gave up, and the context stays usable.  Plus the
KV push kernel with an out-of-range block id (recorded and skipped, not accessed)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_runs_out_and_reports_status():
    from omni_infer_b200.ops import _native as nat
    from omni_infer_b200.parallel.ep_fused import EpLayout, _align

    L = nat.lib()
    dev = torch.device("cuda")
    # a two-rank layout emulated in one buffer: "rank 1" never sends, so its flag stays 0
    W, cap, H, slots = 2, 8, 128, 8
    lay = EpLayout(world=W, rank=0, cap=cap, H=H, max_slots=slots)
    off = 0
    for name, size in (("off_recv_x", W * cap * H), ("off_recv_s", W * cap * 4), ("off_recv_meta", W * cap * 16),
                       ("off_recv_cnt", 256), ("off_recv_flag", 256), ("off_comb", slots * H * 2), ("off_comb_flag", 256),
                       ("off_ctrl", 256)):
        setattr(lay, name, off)
        off = _align(off + size)
    buf = torch.zeros(off, dtype=torch.uint8, device=dev)
    ctrl = buf[lay.off_ctrl:lay.off_ctrl + 8].view(torch.int32)
    ctrl[0] = 1                                                   # the round whose flags are awaited
    buf[lay.off_recv_flag:lay.off_recv_flag + 4].view(torch.int32)[0] = 1   # own flag arrived, peer's did not
    peers = (ctypes.c_void_p * 16)(*([ctypes.c_void_p(buf.data_ptr())] * 2 + [None] * 14))
    n = W * cap
    ids = torch.empty(n, dtype=torch.int32, device=dev)
    w = torch.empty(n, dtype=torch.float32, device=dev)
    slot = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.full((W,), -5, dtype=torch.int32, device=dev)
    status = nat.status_buffer(dev)
    status.zero_()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = L.omni_ep_dispatch_recv(ctypes.byref(lay), peers, nat.ptr(ids), nat.ptr(w), nat.ptr(slot), nat.ptr(counts),
                                 ctypes.c_ulonglong(2_000_000), nat.ptr(status), nat.stream())   # 2 ms limit
    t1.record()
    torch.cuda.synchronize()
    assert rc == 0
    assert t0.elapsed_time(t1) < 500.0                            # it gave up by itself
    code, site, _, detail = status.tolist()
    assert code == 2 and site == 201 and detail == 1              # flag timeout, dispatch receive, peer 1
    assert counts.tolist() == [0, 0] and (ids == -1).all()        # nothing was taken from the silent peer
    # the status word is still set (the host has not read it): the next wait on the silent peer, with a limit of a
    # whole second, gives up at once instead of spending its own limit, so a lost peer costs one limit per step and
    # not one per layer
    t2 = torch.cuda.Event(enable_timing=True); t3 = torch.cuda.Event(enable_timing=True)
    t2.record()
    rc = L.omni_ep_dispatch_recv(ctypes.byref(lay), peers, nat.ptr(ids), nat.ptr(w), nat.ptr(slot), nat.ptr(counts),
                                 ctypes.c_ulonglong(1_000_000_000), nat.ptr(status), nat.stream())
    t3.record()
    torch.cuda.synchronize()
    assert rc == 0 and t2.elapsed_time(t3) < 100.0
    assert status.tolist()[:2] == [2, 201]                        # the first record is kept
    with pytest.raises(nat.KernelProtocolError):
        nat.check_status()
    # the context is still fine
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0
    nat.check_status()


def test_kv_push_copies_blocks_and_rejects_bad_ids():
    from omni_infer_b200.accelerators.pd.kv_push import PeerCacheView, push_blocks_cuda
    from omni_infer_b200.ops import _native as nat

    dev = "cuda"
    src = [torch.randn(10, 16, 576, device=dev).bfloat16() for _ in range(3)]
    dst = [torch.zeros(12, 16, 576, device=dev, dtype=torch.bfloat16) for _ in range(3)]
    view = PeerCacheView([t.data_ptr() for t in dst], 16 * 576 * 2, 12)
    push_blocks_cuda(src, view, [1, 4, 9], [11, 0, 5])
    for s, d in zip(src, dst):
        assert torch.equal(d[11], s[1]) and torch.equal(d[0], s[4]) and torch.equal(d[5], s[9])
        assert float(d[1].abs().sum()) == 0
    nat.check_status()
    push_blocks_cuda(src, view, [2], [99])                       # destination block out of range
    torch.cuda.synchronize()
    st = nat.status_buffer().tolist()
    assert st[0] == 3 and st[1] == 300                            # bounds error recorded, access skipped
    nat.status_buffer().zero_()


def test_router_drops_and_reports_a_row_of_nan_scores():
    """A row whose router scores are all NaN has no selectable expert: its pairs come back as id -1 with weight 0, the
    status word names the row, other rows are routed as usual, and nothing is indexed with the invalid id (neither the
    selector table nor the activation histogram)."""
    from omni_infer_b200 import ops
    from omni_infer_b200.ops import _native as nat

    dev = torch.device("cuda")
    T, E, k = 6, 64, 8
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = torch.randn(T, E, device=dev, generator=g)
    logits[3] = float("nan")
    selector = torch.arange(E, dtype=torch.int32, device=dev).flip(0).contiguous()
    counts = torch.zeros(E, dtype=torch.int64, device=dev)
    nat.status_buffer(dev).zero_()
    ids, w = ops.router_topk(logits, k, selector=selector, counts=counts, mode="sigmoid", renorm=True, scale=1.0)
    torch.cuda.synchronize()
    with pytest.raises(nat.KernelProtocolError) as ei:
        nat.check_status()
    assert "code=3" in str(ei.value) and "detail=3" in str(ei.value)
    assert ids[3].tolist() == [-1] * k and w[3].abs().sum().item() == 0.0
    ok = [0, 1, 2, 4, 5]
    ref_ids, _ = ops.router_topk_ref(logits[ok], k, mode="sigmoid", renorm=True, scale=1.0)
    assert torch.equal(ids[ok].sort(-1).values.long(), (E - 1 - ref_ids.long()).sort(-1).values)
    assert counts.sum().item() == len(ok) * k
    nat.check_status()                                            # cleared; the context is still usable
