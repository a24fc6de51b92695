#!/usr/bin/env python
"""Headline benchmark: decode throughput of DeepSeek-V3 (block-scaled e4m3 weights, EP-MoE over all
ranks, data-parallel MLA attention, 1 MTP draft layer) served through the engine's public API.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched with torch.distributed.run)

Every rank holds 32 routed experts per MoE layer and decodes 256 sequences (weak scaling).  With 8 ranks
this is the full 256-expert DeepSeek-V3-671B; with fewer ranks the model has 32*N routed experts (the
671B checkpoint does not fit on fewer than 8 GPUs) and the JSON line says so.  Random-init weights,
uniform random token ids.  ``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="deepseek-v3", choices=["deepseek-v3", "deepseek-v2-lite", "qwen3-30b-a3b", "small"])
    ap.add_argument("--batch", type=int, default=0, help="decode sequences per GPU (default: the config's)")
    ap.add_argument("--input-len", type=int, default=0)
    ap.add_argument("--mtp", type=int, default=-1, help="speculative tokens (default: the config's)")
    ap.add_argument("--accept-rate", type=float, default=-1.0, help="force the MTP acceptance rate (test knob)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (the result is then not a benchmark)")
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--ep-backend", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--attn-tp", action="store_true",
                    help="tensor-parallel attention over all ranks (one shared batch) instead of data-parallel attention")
    ap.add_argument("--tp-backend", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--synthetic-kv", action="store_true", help="fill the KV cache without running prefill")
    return ap.parse_args()


def reference_arm(args):
    """The reference is a set of plugins for vLLM 0.9.0 on Ascend NPUs: its package installs
    (pip --no-deps into baseline/_ref) but importing its platform needs torch_npu / CANN and vLLM 0.9.0
    internals; every device op is a closed Ascend library call and every collective is HCCL."""
    why = "reference is Ascend-only (torch_npu/CANN ops, HCCL, vLLM 0.9.0 plugin ABI); installs with --no-deps but cannot import or run on CUDA"
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import importlib
        importlib.import_module("omni.adaptors.vllm.platform")
        why = "reference platform imported but has no CUDA device path (all ops are torch_npu calls)"
    except Exception as e:  # noqa: BLE001
        why += f" [{type(e).__name__}: {str(e)[:80]}]"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, col in (("hw_slowdown", 3), ("hw_thermal_slowdown", 4), ("sw_thermal_slowdown", 5), ("sw_power_cap", 6)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist

    from omni_infer_b200.engine.engine_core import EngineConfig, EngineCore
    from omni_infer_b200.engine.request import SamplingParams
    from omni_infer_b200.models.config import get_config
    from omni_infer_b200.ops import _native as nat

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)

    if args.config == "deepseek-v3":
        mc = get_config("deepseek-v3")
        mc.n_routed_experts = 32 * world
        mc.n_group = world
        mc.topk_group = min(4, world)
        batch, in_len, mtp = 256, 2048, 1
        name = "deepseek-v3-671b-fp8" if world == 8 else f"deepseek-v3-fp8 rank-slice ({32 * world} routed experts; full 256-expert model needs 8 GPUs)"
    elif args.config == "deepseek-v2-lite":
        mc = get_config("deepseek-v2-lite")
        batch, in_len, mtp = 128, 1024, 0
        name = "deepseek-v2-lite-bf16"
    elif args.config == "qwen3-30b-a3b":
        mc = get_config("qwen3-30b-a3b")
        batch, in_len, mtp = 128, 4096, 0
        name = "qwen3-30b-a3b-bf16"
    else:
        mc = get_config("small-deepseek", num_nextn_predict_layers=1)
        batch, in_len, mtp = 32, 256, 1
        name = "small-deepseek"
    if args.layers:
        mc.num_hidden_layers = args.layers
        name += f" [DEBUG {args.layers} layers]"
    batch = args.batch or batch
    in_len = args.input_len or in_len
    mtp = mtp if args.mtp < 0 else args.mtp
    if mtp and mc.num_nextn_predict_layers == 0:
        mtp = 0
    tpr = 1 + mtp
    bs = 128
    total_steps = args.warmup + args.steps
    per_req_tokens = in_len + tpr * (total_steps + 4) + 8
    blocks = batch * ((per_req_tokens + bs - 1) // bs + 1) + 2
    ecfg = EngineConfig(model=mc.name, block_size=bs, num_kv_blocks=blocks, max_num_seqs=batch,
                        max_num_batched_tokens=max(16384, in_len), max_model_len=per_req_tokens + bs,
                        num_speculative_tokens=mtp, decode_gear_list=[batch], enforce_eager=args.eager,
                        seed=1234 + (0 if args.attn_tp else rank), ep_backend=args.ep_backend, attn_tp=args.attn_tp,
                        tp_backend=args.tp_backend)
    t_load = time.time()
    eng = EngineCore(ecfg, model_cfg=mc)
    eng.worker.runner.cfg.control_accept_rate = args.accept_rate
    load_s = time.time() - t_load

    dev = torch.device("cuda", local_rank)
    g = torch.Generator().manual_seed(100 + (0 if args.attn_tp else rank))   # TP attention: every rank serves the same batch
    # the step's inputs start in pinned host memory, as a serving front end would hand them over
    prompts = torch.randint(0, mc.vocab_size, (batch, in_len), generator=g).pin_memory()
    sp = SamplingParams(max_tokens=10 ** 6, ignore_eos=True)

    def barrier():
        if world > 1:
            dist.barrier()

    # ---- prefill (untimed set-up for the decode measurement; also yields TTFT samples)
    ttft = []
    n_single = min(3, batch)
    for i in range(n_single):
        t0 = time.perf_counter()
        eng.add_request(prompts[i].tolist(), sp)
        eng.step()
        torch.cuda.synchronize()
        ttft.append((time.perf_counter() - t0) * 1e3)
    for i in range(n_single, batch):
        eng.add_request(prompts[i].tolist(), sp)
    while eng.scheduler.num_waiting:
        eng.step()
    torch.cuda.synchronize()
    nat.check_status()

    # ---- decode: W warm-up steps, K timed steps
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = nat.launch_count()
    tokens0 = eng.metrics["generated_tokens"]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    step_wall = []
    h2d = d2h = 0
    torch.cuda.synchronize()
    barrier()
    torch.cuda.profiler.start()        # no-op unless a profiler asked for --profile-from-start off
    t_wall0 = time.perf_counter()
    ev[0].record()
    for i in range(args.steps):
        ts = time.perf_counter()
        eng.step()                      # schedule -> H2D inputs -> graph replay -> sample -> D2H tokens
        ev[i + 1].record()
        step_wall.append((time.perf_counter() - ts) * 1e3)
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall0
    torch.cuda.profiler.stop()
    barrier()
    clocks = sampler.stop()
    dev_ms = ev[0].elapsed_time(ev[-1])
    step_dev = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    tokens = eng.metrics["generated_tokens"] - tokens0
    launches = nat.launch_count() - launches0
    nat.check_status()
    # bytes moved per step by the runner: ids, positions, slots (int64), q_seq_lens, seq_lens, q_to_seq, block table (int32)
    n_rows = batch * tpr
    bt_w = eng.worker.runner._bt_width
    h2d = n_rows * 8 * 3 + n_rows * 4 * 2 + batch * 4 + batch * bt_w * 4
    d2h = n_rows * 8 + (batch * mtp * 8 if mtp else 0)

    t = torch.tensor([dev_ms, t_wall * 1e3, float(tokens)], dtype=torch.float64, device=dev)
    if world > 1:
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dev_ms, wall_ms, tokens_total = float(mx[0]), float(mx[1]), float(sm[2])
        if args.attn_tp:
            tokens_total /= world      # one shared batch, counted once
    else:
        dev_ms, wall_ms, tokens_total = float(t[0]), float(t[1]), float(t[2])
    if rank == 0:
        value = tokens_total / (dev_ms / 1e3)
        e2e = tokens_total / (wall_ms / 1e3)
        line = {
            "metric": "decode tok/s/GPU + p50 TPOT/TTFT, DeepSeek-V3 fp8 EP8 (device-timed, max rank)",
            "value": round(value, 1), "unit": "tok/s (all GPUs)", "per_gpu_tok_s": round(value / world, 1),
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 3),
            "tpot_p50_ms": round(statistics.median(step_dev), 3), "ttft_p50_ms": round(statistics.median(ttft), 2),
            "higher_is_better": True, "scaling": "strong" if args.attn_tp else "weak", "vs_baseline": None, "dtype": "fp8_e4m3 weights (128x128 block scales), bf16 activations/KV" if mc.quantization == "fp8_block" else "bf16",
            "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": name, "global_batch": batch * (1 if args.attn_tp else world), "seq_len": in_len, "output_steps": total_steps,
                       "parallelism": (f"tp{world}-attn({args.tp_backend})+ep{world}" if args.attn_tp and world > 1
                                       else f"ep{world}+dp{world}-attn"), "mtp_draft_layers": mtp,
                       "mtp_accepted_tokens_per_step": round(tokens_total / (args.steps * batch * (1 if args.attn_tp else world)), 3),
                       "accept_rate_forced": args.accept_rate, "layers": mc.num_hidden_layers,
                       "routed_experts": mc.n_routed_experts, "cuda_graph": eng.worker.runner.graphs is not None,
                       "l2_policy": "inputs larger than L2 (>= 90 GB of weights and KV streamed per step)",
                       "ep_backend": args.ep_backend if world > 1 else "local", "load_s": round(load_s, 1)},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tok/s (all GPUs)", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "tpot_p50_ms_wall": round(statistics.median(step_wall), 3)},
            "gpu_launches": int(launches),
            "impl": "ours",
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
