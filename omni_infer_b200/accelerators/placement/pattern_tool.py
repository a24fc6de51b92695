"""Offline placement-pattern tool (reference: accelerators/placement/utils/omni_pattern_tool/step_1..4, pipeline.py).

    python -m omni_infer_b200.accelerators.placement.pattern_tool pipeline --inputs DIR --world 8 \
           --redundant-per-rank 4 --workdir out/
    python -m omni_infer_b200.accelerators.placement.pattern_tool --dumps DIR --world 8 --redundant-per-rank 4 \
           --out pattern.npy                                   (one-shot form: steps 1 to 4 without the files between)

Sub-commands, one per step of the reference's pipeline, each reading the previous one's file:

``logs-to-csv``  activation logs (``[dump activation] <prefill|decode> step S in rank R for layer L get N experts data: ...``
                 lines) or folders of dump text files -> one CSV ``layer, ep_0 .. ep_{E-1}`` of summed counts, filtered by
                 mode and step range, optionally in 128-token tiles (ceil), as step 1 of the reference does.
``generate``     CSV -> pattern ``[world, layers, experts]`` .npy, ``rearrange`` (no replica, balanced buckets) or
                 ``redundant`` (C++ ``ExpertLoadBalancer``: load-per-replica max-heap, then LPT with host interleave);
                 ``--special-layers K`` treats only the K most imbalanced layers and leaves the others on the base layout.
``check``        validates a pattern and writes a text view (per layer and rank: the expert ids, replicas marked).
``analyse``      per-layer, per-rank expected load of the base layout and of each pattern as CSV, with the max-load
                 reduction and the max/mean ratio per layer.
``plan``         incremental: current pattern + counts -> at most ``--diff-limit`` instructions per layer as JSON (the
                 static balancer's snapshot planner), for a deployment that cannot afford a whole new pattern.
``pipeline``     all four steps into ``--workdir``."""
from __future__ import annotations

import argparse
import csv
import ctypes
import glob
import json
import math
import os
import re

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


def _legacy_main(argv=None) -> int:
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


# ------------------------------------------------------------------------------------------------ step 1: logs -> CSV
LOG_LINE = re.compile(r"\[dump activation\] (prefill|decode) step (\d+) in rank (\d+) for layer (\d+) get (\d+) experts data: ([\d\s]+)")


def parse_step_range(text):
    if not text:
        return None
    lo, _, hi = text.partition(":")
    lo, hi = int(lo), int(hi)
    if lo > hi:
        raise ValueError(f"step range {text!r}: start after end")
    return lo, hi


def counts_from_logs(paths, layers: int, world: int, per_rank: int, modes=("prefill", "decode"), step_range=None,
                     tile: int = 0) -> np.ndarray:
    """[layers, world * per_rank] summed counts from activation log lines; malformed or out-of-range lines are skipped
    and counted in the returned array's ``skipped`` attribute (a plain int on a ndarray subclass would be lost on
    arithmetic, so the count is returned alongside)."""
    out = np.zeros((layers, world * per_rank), dtype=np.float64)
    skipped = 0
    for path in paths:
        with open(path, errors="replace") as f:
            for line in f:
                m = LOG_LINE.search(line)
                if not m:
                    continue
                mode, step, rank, layer, n, data = m.groups()
                step, rank, layer, n = int(step), int(rank), int(layer), int(n)
                vals = data.split()
                if (mode not in modes or (step_range and not step_range[0] <= step <= step_range[1])):
                    continue
                if not (0 <= rank < world and 0 <= layer < layers) or n != per_rank or len(vals) != n:
                    skipped += 1
                    continue
                v = np.asarray(vals, dtype=np.float64)
                out[layer, rank * per_rank:(rank + 1) * per_rank] += np.ceil(v / tile) if tile else v
    counts_from_logs.last_skipped = skipped
    return out


def counts_from_folders(folders, layers=None, tile: int = 0) -> np.ndarray:
    paths = []
    for d in folders:
        paths += sorted(glob.glob(os.path.join(d, "*.txt"))) if os.path.isdir(d) else sorted(glob.glob(d))
    tot = None
    for p in paths:
        a = np.loadtxt(p, dtype=np.float64, ndmin=2)
        a = np.ceil(a / tile) if tile else a
        tot = a if tot is None else tot + a
    if tot is None:
        raise ValueError("no activation dumps found")
    return tot[:layers] if layers else tot


def write_csv(counts: np.ndarray, path: str) -> None:
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["layer"] + [f"ep_{i}" for i in range(counts.shape[1])])
        for l, row in enumerate(counts):
            w.writerow([l] + [int(x) if float(x).is_integer() else float(x) for x in row])


def read_csv(path: str) -> np.ndarray:
    with open(path, newline="") as f:
        rows = list(csv.reader(f))
    if not rows or rows[0][0] != "layer":
        raise ValueError(f"{path}: not a layer / ep_i table")
    return np.asarray([[float(x) for x in r[1:]] for r in rows[1:]], dtype=np.float64)


# ------------------------------------------------------------------------------------------------ step 2: CSV -> pattern
def layer_imbalance(loads: np.ndarray, world: int) -> np.ndarray:
    """max/mean rank load of the base layout (expert e on rank e // (E / world)), per layer."""
    layers, experts = loads.shape
    rl = loads.reshape(layers, world, experts // world).sum(axis=2)
    return rl.max(axis=1) / rl.mean(axis=1).clip(min=1e-9)


def rearrange_layer(loads_row: np.ndarray, world: int) -> np.ndarray:
    """No replica: experts sorted by load, dealt onto the currently lightest rank that still has room."""
    experts = loads_row.shape[0]
    per = experts // world
    order = np.argsort(-loads_row, kind="stable")
    rl, used = np.zeros(world), np.zeros(world, dtype=np.int64)
    place = np.full(world * per, -1, dtype=np.int32)
    for e in order:
        open_ranks = np.nonzero(used < per)[0]
        r = open_ranks[np.argmin(rl[open_ranks])]
        place[r * per + used[r]] = e
        used[r] += 1
        rl[r] += loads_row[e]
    return place


def generate(loads: np.ndarray, world: int, mode: str = "redundant", redundant_per_rank: int = 0, special_layers: int = -1,
             max_redundant_per_expert: int = 10, ranks_per_host: int = 8) -> np.ndarray:
    layers, experts = loads.shape
    if experts % world:
        raise ValueError("experts must divide evenly over the ranks")
    if mode not in ("rearrange", "redundant"):
        raise ValueError("mode is rearrange or redundant")
    red = redundant_per_rank if mode == "redundant" else 0
    slots = experts // world + red
    base = np.full((layers, world * slots), -1, dtype=np.int32)
    per = experts // world
    for r in range(world):
        base[:, r * slots:r * slots + per] = np.arange(r * per, (r + 1) * per)
    chosen = np.arange(layers)
    if 0 <= special_layers < layers:
        chosen = np.argsort(-layer_imbalance(loads, world), kind="stable")[:special_layers]
    placement = base.copy()
    if mode == "redundant":
        full = pattern_to_placement(generate_pattern(loads, world, red, max_redundant_per_expert, ranks_per_host), slots)
        placement[chosen] = full[chosen]
    else:
        for l in chosen:
            placement[l] = rearrange_layer(loads[l], world)
    return pattern_from_placement(placement, world, slots, experts)


def pattern_to_placement(pattern: np.ndarray, slots: int | None = None) -> np.ndarray:
    world, layers, experts = pattern.shape
    slots = slots or int(pattern.sum(axis=2).max())
    out = np.full((layers, world * slots), -1, dtype=np.int32)
    for r in range(world):
        for l in range(layers):
            ids = np.nonzero(pattern[r, l])[0]
            out[l, r * slots:r * slots + len(ids)] = ids
    return out


# ------------------------------------------------------------------------------------------------ step 3: check + view
def pattern_view(pattern: np.ndarray) -> str:
    world, layers, experts = pattern.shape
    reps = pattern.sum(axis=0)
    lines = [f"# {world} ranks, {layers} layers, {experts} experts; * marks an expert with more than one replica"]
    for l in range(layers):
        lines.append(f"layer {l}: {int((reps[l] > 1).sum())} replicated experts, {int(pattern[:, l].sum())} slots in use")
        for r in range(world):
            ids = np.nonzero(pattern[r, l])[0]
            lines.append(f"  rank {r}: " + " ".join(f"{e}{'*' if reps[l, e] > 1 else ''}" for e in ids))
    return "\n".join(lines) + "\n"


# ------------------------------------------------------------------------------------------------ step 4: analysis
def rank_loads(pattern: np.ndarray, loads: np.ndarray) -> np.ndarray:
    """[layers, world] expected load when every expert's load is split evenly over its replicas."""
    reps = pattern.sum(axis=0).clip(min=1)
    return (pattern * (loads / reps)[None]).sum(axis=2).T


def analyse_table(patterns: dict, loads: np.ndarray, world: int) -> list:
    """One row per (layer, deployment): per-rank loads, the best possible load (total / world), the max load, the
    max/mean ratio and the reduction of the max load against the base layout."""
    layers, experts = loads.shape
    deployments = {"base": base_pattern(world, layers, experts), **patterns}
    base_max = rank_loads(deployments["base"], loads).max(axis=1)
    rows = []
    for name, pat in deployments.items():
        rl = rank_loads(pat, loads)
        for l in range(layers):
            best = loads[l].sum() / world
            mx = rl[l].max()
            rows.append({"deployment": name, "layer": l, **{f"rank_{r}": float(rl[l, r]) for r in range(world)},
                         "best": float(best), "max": float(mx), "max_over_mean": float(mx / max(rl[l].mean(), 1e-9)),
                         "max_load_reduction": float(1.0 - mx / base_max[l]) if base_max[l] > 0 else 0.0})
    return rows


def write_rows(rows: list, path: str) -> None:
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
        w.writeheader()
        w.writerows(rows)


# ------------------------------------------------------------------------------------------------ incremental plan
OP_NAMES = {0: "swap", 1: "add", 2: "remove", 3: "empty"}


def plan_instructions(placement: np.ndarray, counts: np.ndarray, world: int, experts: int, diff_limit: int = -1,
                      max_redundant_per_expert: int = 10, accept_margin: float = 0.1, ranks_per_host: int = 8):
    """placement / counts: [layers, world * slots] (expert id or -1; activations per position).  Returns the list of
    instruction dicts in execution order and a [layers, 2] array of the simulated max/mean ratio before and after."""
    layers, positions = placement.shape
    slots = positions // world
    pl = np.ascontiguousarray(placement, dtype=np.int32)
    ac = np.ascontiguousarray(counts, dtype=np.int64)
    cap = layers * max(positions, 1) * 2 + 16
    out = np.zeros((cap, 9), dtype=np.int32)
    ratios = np.zeros((layers, 2), dtype=np.float64)
    n = nat.lib().omni_pl_static_instructions(pl.ctypes.data, ac.ctypes.data, layers, world, experts, slots, ranks_per_host,
                                              max_redundant_per_expert, diff_limit, accept_margin, out.ctypes.data, cap,
                                              ratios.ctypes.data)
    if n < 0:
        raise RuntimeError("the static planner rejected the input (see stderr)")
    keys = ("layer", "op", "source_rank", "source_expert", "source_position", "target_rank", "target_expert",
            "target_position", "wave")
    ins = [{k: (OP_NAMES[int(v)] if k == "op" else int(v)) for k, v in zip(keys, row)} for row in out[:n]]
    return ins, ratios


# ------------------------------------------------------------------------------------------------ CLI
def _load_counts(a) -> np.ndarray:
    step_range = parse_step_range(a.step_range)
    modes = ("prefill", "decode") if a.collecting_mode == "all" else (a.collecting_mode,)
    if a.input_mode == "log":
        if not (a.layers and a.world_of_data and a.positions):
            raise SystemExit("--input-mode log needs --layers, --world-of-data and --positions")
        return counts_from_logs(a.inputs, a.layers, a.world_of_data, a.positions // a.world_of_data, modes, step_range, a.tile)
    return counts_from_folders(a.inputs, a.layers or None, a.tile)


def _add_input_args(ap):
    ap.add_argument("--inputs", nargs="+", required=True, help="log files (--input-mode log) or dump folders / globs (txt)")
    ap.add_argument("--input-mode", choices=("log", "txt"), default="txt")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--world-of-data", type=int, default=0, help="ranks of the deployment that produced the logs")
    ap.add_argument("--positions", type=int, default=0, help="expert positions of that deployment (all ranks)")
    ap.add_argument("--collecting-mode", choices=("prefill", "decode", "all"), default="all")
    ap.add_argument("--step-range", default="", help="start:end of the steps to keep")
    ap.add_argument("--tile", type=int, default=0, help="count in tiles of this many tokens (ceil); 0 keeps raw counts")


def _add_generate_args(ap):
    ap.add_argument("--world", type=int, required=True, help="ranks of the target pattern")
    ap.add_argument("--mode", choices=("rearrange", "redundant", "all"), default="redundant")
    ap.add_argument("--redundant-per-rank", type=int, default=1)
    ap.add_argument("--special-layers", type=int, nargs="*", default=[-1],
                    help="treat only the K most imbalanced layers (one pattern per K; -1 = every layer)")
    ap.add_argument("--max-redundant-per-expert", type=int, default=10)
    ap.add_argument("--ranks-per-host", type=int, default=8)


def _generate_all(loads, a, outdir, prefix) -> dict:
    out = {}
    modes = ("rearrange", "redundant") if a.mode == "all" else (a.mode,)
    for mode in modes:
        for k in a.special_layers:
            pat = generate(loads, a.world, mode, a.redundant_per_rank, k, a.max_redundant_per_expert, a.ranks_per_host)
            check_pattern(pat, a.redundant_per_rank if mode == "redundant" else 0)
            name = f"{prefix}_{mode}_{'all' if k < 0 else k}layers_{a.world}ranks"
            np.save(os.path.join(outdir, name + ".npy"), pat)
            out[name] = pat
    return out


def main(argv=None) -> int:
    argv = list(os.sys.argv[1:] if argv is None else argv)
    cmds = ("logs-to-csv", "generate", "check", "analyse", "plan", "pipeline")
    if not argv or argv[0] not in cmds:
        return _legacy_main(argv)
    cmd, argv = argv[0], argv[1:]
    ap = argparse.ArgumentParser(prog=f"pattern_tool {cmd}")
    if cmd == "logs-to-csv":
        _add_input_args(ap)
        ap.add_argument("--out", required=True)
        a = ap.parse_args(argv)
        counts = _load_counts(a)
        write_csv(counts, a.out)
        print(json.dumps({"csv": a.out, "layers": int(counts.shape[0]), "columns": int(counts.shape[1]),
                          "skipped_lines": int(getattr(counts_from_logs, "last_skipped", 0))}))
    elif cmd == "generate":
        ap.add_argument("--csv", required=True)
        ap.add_argument("--outdir", required=True)
        ap.add_argument("--prefix", default="pattern")
        _add_generate_args(ap)
        a = ap.parse_args(argv)
        os.makedirs(a.outdir, exist_ok=True)
        pats = _generate_all(read_csv(a.csv), a, a.outdir, a.prefix)
        print(json.dumps({"patterns": sorted(pats)}))
    elif cmd == "check":
        ap.add_argument("--pattern", required=True)
        ap.add_argument("--redundant-per-rank", type=int, default=0)
        ap.add_argument("--view", default="", help="write the text view here")
        a = ap.parse_args(argv)
        pat = np.load(a.pattern)
        check_pattern(pat, a.redundant_per_rank)
        if a.view:
            with open(a.view, "w") as f:
                f.write(pattern_view(pat))
        print(json.dumps({"ok": True, "shape": list(pat.shape), "replicated": int((pat.sum(axis=0) > 1).sum())}))
    elif cmd == "analyse":
        ap.add_argument("--csv", required=True)
        ap.add_argument("--patterns", nargs="+", required=True)
        ap.add_argument("--out", required=True)
        a = ap.parse_args(argv)
        loads = read_csv(a.csv)
        pats = {os.path.splitext(os.path.basename(p))[0]: np.load(p) for p in a.patterns}
        world = next(iter(pats.values())).shape[0]
        rows = analyse_table(pats, loads, world)
        write_rows(rows, a.out)
        summary = {}
        for r in rows:
            summary.setdefault(r["deployment"], []).append(r["max_over_mean"])
        print(json.dumps({"out": a.out, "mean_max_over_mean": {k: float(np.mean(v)) for k, v in summary.items()}}))
    elif cmd == "plan":
        ap.add_argument("--current-pattern", required=True)
        ap.add_argument("--dumps", required=True, help="folder of per-position dump text files taken under that pattern")
        ap.add_argument("--diff-limit", type=int, default=-1)
        ap.add_argument("--max-redundant-per-expert", type=int, default=10)
        ap.add_argument("--accept-margin", type=float, default=0.1)
        ap.add_argument("--ranks-per-host", type=int, default=8)
        ap.add_argument("--slots", type=int, default=0, help="slots per rank (default: the fullest rank of the pattern)")
        ap.add_argument("--out", required=True)
        a = ap.parse_args(argv)
        cur = np.load(a.current_pattern)
        world, layers, experts = cur.shape
        placement = pattern_to_placement(cur, a.slots or None)
        counts = counts_from_folders([a.dumps], layers)
        if counts.shape != placement.shape:
            raise SystemExit(f"dumps are {counts.shape}, the pattern has {placement.shape} positions")
        ins, ratios = plan_instructions(placement, counts, world, experts, a.diff_limit, a.max_redundant_per_expert,
                                        a.accept_margin, a.ranks_per_host)
        with open(a.out, "w") as f:
            json.dump({"instructions": ins, "ratio_before": ratios[:, 0].tolist(), "ratio_after": ratios[:, 1].tolist()}, f)
        print(json.dumps({"out": a.out, "instructions": len(ins), "mean_ratio_before": float(ratios[:, 0].mean()),
                          "mean_ratio_after": float(ratios[:, 1].mean())}))
    else:   # pipeline
        _add_input_args(ap)
        _add_generate_args(ap)
        ap.add_argument("--workdir", required=True)
        ap.add_argument("--prefix", default="pattern")
        a = ap.parse_args(argv)
        os.makedirs(a.workdir, exist_ok=True)
        counts = _load_counts(a)
        csv_path = os.path.join(a.workdir, "topk_id_count.csv")
        write_csv(counts, csv_path)
        loads = read_csv(csv_path)
        pats = _generate_all(loads, a, a.workdir, a.prefix)
        for name, pat in pats.items():
            with open(os.path.join(a.workdir, name + ".view.txt"), "w") as f:
                f.write(pattern_view(pat))
        rows = analyse_table(pats, loads, a.world)
        write_rows(rows, os.path.join(a.workdir, "load_analysis.csv"))
        summary = {}
        for r in rows:
            summary.setdefault(r["deployment"], []).append(r["max_over_mean"])
        print(json.dumps({"workdir": a.workdir, "patterns": sorted(pats),
                          "mean_max_over_mean": {k: float(np.mean(v)) for k, v in summary.items()}}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
