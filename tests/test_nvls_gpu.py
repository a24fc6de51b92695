"""In-switch reduction (multimem over an NVSwitch multicast mapping) on 2+ GPUs: the all-reduce and the fused
reduce-scatter + residual + RMSNorm against NCCL / fp32 references, replay from a CUDA graph, and device-timed
comparison with NCCL.  Every rank stays until the end (a rank that leaves while bound to a multicast object would
disturb its peers), so nothing here injects a failure."""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, json, torch
sys.path.insert(0, os.environ["OMNI_ROOT"])
import torch.distributed as dist
from omni_infer_b200 import ops
from omni_infer_b200.ops import _native as nat
from omni_infer_b200.parallel import nvls
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); lr = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(lr)
dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
grp = dist.group.WORLD
res = {"world": world}
if not nvls.available():
    res["skipped"] = "no multicast support on this device / driver"
else:
    ws = nvls.NvlsWorkspace(grp, 64 << 20)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    # ---- all-reduce numerics (fp32 sum over ranks as the reference)
    x = (torch.randn(512, 7168, generator=g, device="cuda") * 0.5).bfloat16()
    want = x.float().clone()
    dist.all_reduce(want)
    got = ws.all_reduce(x)
    res["allreduce_max_err"] = float((got.float() - want).abs().max())
    res["allreduce_ref_max"] = float(want.abs().max())
    # ---- reduce rows + residual + RMSNorm
    T, N = 64 * world, 2048
    part = (torch.randn(T, N, generator=g, device="cuda") * 0.3).bfloat16()
    tot = part.float().clone()
    dist.all_reduce(tot)
    rpr = T // world
    resid = (torch.randn(rpr, N, generator=g, device="cuda") * 0.2).bfloat16()
    wn = (torch.rand(N, generator=g, device="cuda") + 0.5).bfloat16()
    ws.view((T, N)).copy_(part)
    out, normed = ws.reduce_rows(T, N, residual=resid, norm_weight=wn, eps=1e-6)
    ref_sum = (tot[rank * rpr:(rank + 1) * rpr] + resid.float())
    res["rows_max_err"] = float((out.float() - ref_sum).abs().max())
    rs = ref_sum.bfloat16().float()
    ref_norm = rs * torch.rsqrt(rs.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()
    res["norm_max_err"] = float((normed.float() - ref_norm).abs().max())
    # ---- replay from a CUDA graph with new inputs each time
    n_el = 256 * 2048
    v = ws.view((n_el,))
    src = torch.zeros(n_el, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        v.copy_(src); ws.all_reduce_(n_el)          # warm-up outside capture
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize(); dist.barrier()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        v.copy_(src)
        ws.all_reduce_(n_el)
    ok = True
    for it in range(3):
        src.fill_(float(rank + 1 + it))
        gr.replay()
        torch.cuda.synchronize()
        ok = ok and bool((v.float() == float(sum(r + 1 + it for r in range(world)))).all())
    res["graph_replay_ok"] = ok
    nat.check_status()
    # ---- timing against NCCL (device events, max over ranks), in place on both sides
    times = {}
    for nbytes in (256 << 10, 4 << 20, 64 << 20):
        n_el = nbytes // 2
        t = torch.ones(n_el, dtype=torch.bfloat16, device="cuda")
        ws.view((n_el,)).fill_(1.0)
        row = {}
        for name, fn in (("nvls", lambda: ws.all_reduce_(n_el)), ("nccl", lambda: dist.all_reduce(t))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize(); dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            iters = 20
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            row[name + "_us"] = round(float(ms) * 1e3, 1)
        row["busbw_nvls_gbs"] = round(2 * (world - 1) / world * nbytes / (row["nvls_us"] * 1e-6) / 1e9, 1)
        row["busbw_nccl_gbs"] = round(2 * (world - 1) / world * nbytes / (row["nccl_us"] * 1e-6) / 1e9, 1)
        times[str(nbytes)] = row
    res["timing"] = times
    nat.check_status()
torch.cuda.synchronize()
dist.barrier()
if rank == 0:
    print("RESULT " + json.dumps(res))
dist.destroy_process_group()
'''


def _run(world, port):
    env = dict(os.environ, OMNI_ROOT=ROOT)
    with tempfile.NamedTemporaryFile("w", suffix="_nvls_worker.py", delete=False) as f:
        f.write(WORKER)
        script = f.name
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), script]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    os.unlink(script)
    if res.returncode != 0:
        errs = [l for l in res.stderr.splitlines() if not l.startswith(("W1", "[W", "***")) and "OMP_NUM" not in l]
        raise AssertionError("\n".join(res.stdout.splitlines()[-10:] + errs[-40:]))
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_in_switch_all_reduce_and_reduce_rows():
    world = min(torch.cuda.device_count(), 8)
    world = 8 if world >= 8 else (4 if world >= 4 else 2)
    r = _run(world, 29641)
    if "skipped" in r:
        pytest.skip(r["skipped"])
    print("NVLS", json.dumps(r))
    out = os.environ.get("OMNI_RESULT_DIR", "")      # where to leave the measured timings, if anywhere
    if out and os.path.isdir(out):
        with open(os.path.join(out, f"nvls_allreduce_n{world}.json"), "w") as f:
            json.dump(r, f)
    # bf16 results of sums of `world` values of magnitude ~2: half an ulp of the result
    assert r["allreduce_max_err"] <= r["allreduce_ref_max"] * 2.0 ** -8 + 1e-3, r
    assert r["rows_max_err"] < 0.05 and r["norm_max_err"] < 0.06, r
    assert r["graph_replay_ok"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_attention_with_in_switch_reduction_matches_oracle():
    """The small MLA + MoE model with tensor-parallel attention whose o_proj reduce-scatter (+ residual + RMSNorm) runs
    through the NVSwitch: every generated token against the fp32 oracle, first tokens equal to the peer-store path's."""
    import test_multi_gpu as mg
    from omni_infer_b200.parallel import nvls
    if not nvls.available():
        pytest.skip("no multicast support on this device / driver")
    world = 8 if torch.cuda.device_count() >= 8 else (4 if torch.cuda.device_count() >= 4 else 2)
    env = {"ATTN_TP": "1", "TP_BACKEND": "nvls"}
    # this worker must keep NVLS on: _run of the other file switches it off for NCCL, which does not affect the
    # symmetric-memory rendezvous of the workspace
    got = mg._run(world, env, 29651)
    mg._near_oracle(got, what=f"TP{world} attention, in-switch reduce-scatter")
    peer = mg._run(world, {"ATTN_TP": "1", "TP_BACKEND": "fused"}, 29652)
    assert [o[0] for o in got] == [o[0] for o in peer]
