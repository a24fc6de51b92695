"""Expert-parallel dispatch / combine kernels with four ranks emulated on one GPU (one region of a device buffer per rank,
the ranks' kernels launched one after the other): combine(dispatch(x)) with identity experts must reproduce the
weighted sum of the (quantised) rows.  Covers the three payload paths of the dispatch: quantise in the kernel, copy rows
that are already e4m3, and plain bf16 rows."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("extra", [[], ["--prequant"], ["--payload", "bf16"]])
def test_ep_selfloop_roundtrip(extra):
    cmd = [sys.executable, os.path.join(ROOT, "benchmarks", "ep_selfloop_bench.py"), "--world", "4", "--tokens", "96",
           "--hidden", "1024", "--topk", "4", "--experts-per-rank", "8", "--iters", "1"] + extra
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["rel_err_vs_reference"] < 2e-2
