"""The workload scripts under benchmarks/ run end to end on CPU with tiny sizes (their logic, not their speed)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, NO_GPU_MOCK="1", CUDA_VISIBLE_DEVICES="")


def _run(args):
    res = subprocess.run([sys.executable] + args, capture_output=True, text=True, timeout=600, env=ENV, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])


def test_pd_poisson_workload_finishes_every_request():
    out = _run(["benchmarks/config4_pd_poisson.py", "--config", "small", "--rate", "6", "--duration", "1.5", "--input-len", "40",
                "--output-len", "6", "--max-decode-batch", "8"])
    assert out["finished"] == out["requests"] > 0
    assert out["ttft_ms"]["p50"] > 0 and out["tpot_ms"]["p50"] > 0


def test_placement_stress_workload_reports_load_ratios():
    out = _run(["benchmarks/config5_placement_stress.py", "--config", "small", "--steps", "8", "--batch", "4", "--input-len", "16",
                "--replace-every", "4"])
    for arm in ("baseline", "with_placement"):
        assert out[arm]["tok_s_per_gpu"] > 0
    assert out["with_placement"]["max_over_mean_position_load"] >= 1.0


def test_placement_stress_two_ranks_moves_experts_and_evens_rank_load():
    """Two gloo ranks: the planner must size its tables from the real world size, and a dynamic round must lower the
    rank-load imbalance of the Zipf-biased router."""
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", "29655", "benchmarks/config5_placement_stress.py", "--config", "small",
                          "--steps", "32", "--batch", "4", "--input-len", "16", "--redundant", "2", "--replace-every", "8"],
                         capture_output=True, text=True, timeout=600, env=ENV, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["baseline"]["moves_applied"] == 0 and out["with_placement"]["moves_applied"] > 0
    assert out["with_placement"]["max_over_mean_rank_load"] < out["baseline"]["max_over_mean_rank_load"]
