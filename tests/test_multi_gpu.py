"""Multi-GPU checks (2 ranks as child processes): fused NVLink expert-parallel dispatch/combine against the
single-rank result, the NCCL all-to-all baseline, and the bounded-wait status path.  NVLS is disabled and the
kernels use plain peer loads/stores, so a rank that exits between steps cannot disturb its peers."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, json, torch
sys.path.insert(0, os.environ["OMNI_ROOT"])
import torch.distributed as dist
from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
from omni_infer_b200.engine.request import SamplingParams
from omni_infer_b200.models.config import get_config
from omni_infer_b200.ops import _native as nat
backend = os.environ.get("EP_BACKEND", "fused")
mc = get_config("small-deepseek", quantization="fp8_block", num_nextn_predict_layers=1)
eng = EngineCore(EngineConfig(block_size=128, num_kv_blocks=24, max_model_len=512, max_num_seqs=4,
                              num_speculative_tokens=int(os.environ.get("MTP", "0")), ep_backend=backend, seed=7), model_cfg=mc)
rank = int(os.environ.get("RANK", "0"))
g = torch.Generator().manual_seed(5)
prompts = [torch.randint(0, 4096, (40,), generator=g).tolist() for _ in range(4)]
# data-parallel attention: every rank serves the same four prompts here so results can be compared 1:1
for p in prompts:
    eng.add_request(p, SamplingParams(max_tokens=8))
outs = eng.run_until_done()
torch.cuda.synchronize()
nat.check_status()
if rank == 0:
    print("RESULT " + json.dumps([outs[k] for k in sorted(outs)]))
if dist.is_initialized():
    dist.barrier()
    dist.destroy_process_group()
'''


def _run(world, env_extra, port):
    import tempfile

    env = dict(os.environ, OMNI_ROOT=ROOT, NCCL_NVLS_ENABLE="0", **env_extra)
    with tempfile.NamedTemporaryFile("w", suffix="_ep_worker.py", delete=False) as f:
        f.write(WORKER)
        script = f.name
    if world == 1:
        cmd = [sys.executable, script]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    os.unlink(script)
    if res.returncode != 0:
        errs = [l for l in res.stderr.splitlines() if not l.startswith(("W1", "[W", "***")) and "OMP_NUM" not in l]
        raise AssertionError("\n".join(res.stdout.splitlines()[-10:] + errs[-40:]))
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    import json
    return json.loads(line[len("RESULT "):])


def _agreement(a, b):
    tot = sum(len(x) for x in a)
    same = 0
    for x, y in zip(a, b):
        for u, v in zip(x, y):
            if u != v:
                break
            same += 1
    return same / max(tot, 1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep2_fused_and_nccl_match_single_rank():
    single = _run(1, {}, 0)
    fused = _run(2, {"EP_BACKEND": "fused"}, 29611)
    nccl = _run(2, {"EP_BACKEND": "nccl"}, 29612)
    assert _agreement(fused, single) > 0.6
    assert _agreement(nccl, single) > 0.6
    assert _agreement(fused, nccl) > 0.6
