#!/usr/bin/env python
"""Load-balance stress for OmniPlacement: a fixed per-layer router bias makes expert popularity Zipf-like (s = 1.2 over a
random expert permutation, seed 0).  Runs the same decode workload with and without redundant expert slots and periodic
re-placement, and reports the max/mean expert-position load, the max/mean rank load and the decode throughput.

    python benchmarks/config5_placement_stress.py --config small --steps 64                      # one GPU or CPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/config5_placement_stress.py --config deepseek-v3 --redundant 4 --replace-every 1000 --steps 2048

The reference's counterpart is its placement optimiser fed by recorded activations
(omni/accelerators/placement/omni_placement/omni_planner.py, cpp/placement_manager.cpp)."""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore  # noqa: E402
from omni_infer_b200.engine.request import SamplingParams  # noqa: E402
from omni_infer_b200.models.config import get_config  # noqa: E402


def run(args, redundant: int, dynamic: bool):
    from omni_infer_b200.accelerators.placement import OmniPlanner
    from omni_infer_b200.parallel.parallel_state import get_parallel_state
    mc = get_config("deepseek-v3", quantization="fp8_block") if args.config == "deepseek-v3" else \
        get_config("small-deepseek", quantization="fp8_block" if torch.cuda.is_available() else "none")
    if args.layers:
        mc.num_hidden_layers = args.layers
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.config == "deepseek-v3" and world < 8:
        mc.n_routed_experts = 32 * world          # per-rank slice of the full model (as bench.py does)
        mc.n_group, mc.topk_group = 1, 1
    device = "cuda" if torch.cuda.is_available() else "cpu"
    mc.router_skew = {"s": 1.2, "strength": 6.0, "seed": 0}     # part of the model, so captured decode graphs include it
    # the baseline run also gets a planner (identity placement, never re-placed) so that both runs count loads the same way
    background = dynamic and args.background
    # background: rounds run on the planner's own thread every --period seconds while decode goes on; the runner applies
    # a finished round between two steps (every 16 steps it looks for one).  Otherwise rounds run synchronously below.
    pc = {"max_redundant_per_rank": redundant, "enable_dynamic": background, "period_s": args.period,
          "apply_interval": 16 if background else 10 ** 9}
    bs = 128 if device == "cuda" else 16
    per_req = args.input_len + args.steps + 16
    ecfg = EngineConfig(model=mc.name, block_size=bs, num_kv_blocks=args.batch * (per_req // bs + 2) + 2, max_num_seqs=args.batch,
                        max_model_len=per_req + bs, device=device, seed=3, placement_config=pc,
                        enforce_eager=device == "cpu", decode_gear_list=[args.batch])
    eng = EngineCore(ecfg, model_cfg=mc)
    rank = get_parallel_state().rank
    planner = eng.worker.runner.planner
    g = torch.Generator().manual_seed(7 + rank)
    sp = SamplingParams(max_tokens=10 ** 6, ignore_eos=True)
    for _ in range(args.batch):
        eng.add_request(torch.randint(0, mc.vocab_size, (args.input_len,), generator=g).tolist(), sp)
    while eng.scheduler.num_waiting:
        eng.step()
    if planner is not None:
        planner.sent_counts.zero_()
    moves, rounds, round_s, snap = 0, 0, 0.0, None
    if device == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    tok0 = eng.metrics["generated_tokens"]
    for i in range(args.steps):
        eng.step()
        if planner is not None and (i + 1) % args.replace_every == 0 and i + 1 < args.steps:
            snap = planner.sent_counts.clone()    # the last window starts at the last round boundary, in both arms
        if dynamic and not background and planner is not None and (i + 1) % args.replace_every == 0:
            if device == "cuda":
                torch.cuda.synchronize()
            tr = time.perf_counter()
            planner.run_round()                   # synchronous round: collect, optimise, stage
            moves += planner.apply_pending()      # between steps: copy staged experts, refresh the selector
            if device == "cuda":
                torch.cuda.synchronize()
            round_s += time.perf_counter() - tr
            rounds += 1
    if device == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if device == "cuda":
        from omni_infer_b200.ops import _native as nat
        nat.check_status()
    stats = planner.load_stats()
    if background:
        from omni_infer_b200.accelerators.placement import _native as pnat
        moves = planner.applied_total
        rounds = pnat.lib().omni_pl_placement_rounds(planner._placement) if planner._placement else 0
    res = {"redundant_slots_per_rank": redundant, "dynamic": dynamic, "background_rounds": bool(background),
           "moves_applied": int(moves),
           "tok_s_per_gpu": round((eng.metrics["generated_tokens"] - tok0) / dt, 1),
           # a round runs synchronously here; in serving it runs on the planner's thread once a minute
           "tok_s_per_gpu_outside_rounds": round((eng.metrics["generated_tokens"] - tok0) / max(dt - round_s, 1e-9), 1),
           "rounds": rounds, "ms_per_round": round(round_s / rounds * 1e3, 1) if rounds else None,
           **{k: round(v, 3) for k, v in stats.items()}}
    if planner is not None and snap is not None:
        res["last_window"] = {k: round(v, 3) for k, v in planner.load_stats(since=snap).items()}
    if planner is not None:
        OmniPlanner.cleanup()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="small", choices=["small", "deepseek-v3"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--input-len", type=int, default=64)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--redundant", type=int, default=2, help="redundant expert slots per rank in the second run")
    ap.add_argument("--replace-every", type=int, default=16)
    ap.add_argument("--background", action="store_true", help="placement rounds on the planner's thread while decode runs")
    ap.add_argument("--period", type=float, default=5.0, help="seconds between background rounds")
    a = ap.parse_args()
    out = {"baseline": run(a, 0, False), "with_placement": run(a, a.redundant, True)}
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
