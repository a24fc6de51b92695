"""Offline placement-pattern tool (reference: omni_planner/utils/omni_pattern_tool/step_1..4, pipeline.py).

    python -m omni_infer_b200.accelerators.placement.pattern_tool --dumps DIR --world 8 --redundant-per-rank 4 \
           --out pattern.npy

Step 1 reads activation dumps (one text file per collection: a line per MoE layer with one count per physical
position, or per logical expert), step 2 allocates redundant replicas to the hottest experts and assigns replicas
to ranks (C++ ``ExpertLoadBalancer``: load-per-replica max-heap, then LPT with host interleave), step 3 validates
the pattern, step 4 reports the expected rank-load imbalance before / after."""
from __future__ import annotations

import argparse
import ctypes
import glob
import json
import os

import numpy as np

from . import _native as nat
from .expert_mapping import base_pattern, pattern_from_placement


def load_dumps(paths, layers=None) -> np.ndarray:
    """Sum of all dumps -> [layers, columns]."""
    tot = None
    for p in paths:
        a = np.loadtxt(p, dtype=np.float64, ndmin=2)
        tot = a if tot is None else tot + a
    if tot is None:
        raise ValueError("no activation dumps found")
    return tot[:layers] if layers else tot


def per_expert_loads(counts: np.ndarray, placement: np.ndarray | None, experts: int) -> np.ndarray:
    """Fold per-position counts back to logical experts when the dump was taken with a placement in force."""
    if counts.shape[1] == experts or placement is None:
        return counts[:, :experts]
    out = np.zeros((counts.shape[0], experts))
    for l in range(counts.shape[0]):
        for pos, e in enumerate(placement[l]):
            if e >= 0:
                out[l, e] += counts[l, pos]
    return out


def generate_pattern(loads: np.ndarray, world: int, redundant_per_rank: int, max_redundant_per_expert: int = 10,
                     ranks_per_host: int = 8) -> np.ndarray:
    layers, experts = loads.shape
    slots = experts // world + redundant_per_rank
    L = nat.lib()
    placement = np.zeros((layers, world * slots), dtype=np.int32)
    for l in range(layers):
        row = np.ascontiguousarray(loads[l], dtype=np.float64)
        out = np.zeros(world * slots, dtype=np.int32)
        rc = L.omni_pl_static_placement(row.ctypes.data, world, experts, slots, ranks_per_host, max_redundant_per_expert,
                                        out.ctypes.data)
        if rc != 0:
            raise RuntimeError(f"placement generation failed for layer {l} (code {rc})")
        placement[l] = out
    return pattern_from_placement(placement, world, slots, experts)


def check_pattern(pattern: np.ndarray, redundant_per_rank: int) -> None:
    world, layers, experts = pattern.shape
    assert np.isin(pattern, (0, 1)).all(), "entries must be 0/1"
    assert (pattern.sum(axis=0) >= 1).all(), "an expert has no replica"
    assert (pattern.sum(axis=2) <= experts // world + redundant_per_rank).all(), "a rank exceeds its slots"


def analyse(pattern: np.ndarray, loads: np.ndarray) -> dict:
    """Expected max/mean rank load when every expert's load is split evenly over its replicas."""
    world, layers, experts = pattern.shape
    reps = pattern.sum(axis=0).clip(min=1)                      # [layers, experts]
    rank_load = (pattern * (loads / reps)[None]).sum(axis=2)     # [world, layers]
    ratio = rank_load.max(axis=0) / rank_load.mean(axis=0).clip(min=1e-9)
    return {"max_over_mean_rank_load": float(ratio.mean()), "worst_layer": int(ratio.argmax()), "worst": float(ratio.max())}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dumps", required=True, help="directory (or glob) of activation dump text files")
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--experts", type=int, default=0)
    ap.add_argument("--redundant-per-rank", type=int, default=0)
    ap.add_argument("--max-redundant-per-expert", type=int, default=10)
    ap.add_argument("--ranks-per-host", type=int, default=8)
    ap.add_argument("--current-pattern", default="", help=".npy pattern in force when the dumps were taken")
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    paths = sorted(glob.glob(os.path.join(a.dumps, "*.txt"))) if os.path.isdir(a.dumps) else sorted(glob.glob(a.dumps))
    counts = load_dumps(paths)
    experts = a.experts or counts.shape[1]
    placement = None
    if a.current_pattern:
        cur = np.load(a.current_pattern)
        slots = int(cur.sum(axis=2).max())
        placement = np.full((cur.shape[1], a.world * slots), -1, dtype=np.int32)
        for r in range(a.world):
            for l in range(cur.shape[1]):
                ids = np.nonzero(cur[r, l])[0]
                placement[l, r * slots:r * slots + len(ids)] = ids
    loads = per_expert_loads(counts, placement, experts)
    pattern = generate_pattern(loads, a.world, a.redundant_per_rank, a.max_redundant_per_expert, a.ranks_per_host)
    check_pattern(pattern, a.redundant_per_rank)
    np.save(a.out, pattern)
    before = analyse(base_pattern(a.world, loads.shape[0], experts), loads)
    after = analyse(pattern, loads)
    print(json.dumps({"before": before, "after": after, "out": a.out}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
