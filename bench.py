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
    ap.add_argument("--tp-backend", default="fused", choices=["fused", "nvls", "nccl"])
    ap.add_argument("--decode-ctx", type=int, default=-1,
                    help="context length at the middle of the timed steps; -1 = the config's mean decode context "
                         "(input + output / 2), 0 = time right after the prefill")
    ap.add_argument("--no-breakdown", action="store_true", help="skip the untimed per-module timing step")
    ap.add_argument("--no-nccl-arm", action="store_true", help="skip the untimed NCCL all-to-all comparison steps (N > 1)")
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


def fast_forward(eng, n_tokens: int, vocab: int, seed: int) -> None:
    """Advance every running request by ``n_tokens`` without running the model: synthetic output ids, KV slots
    allocated by the block manager and filled with random values in every layer's cache.  The timed decode steps
    then run at the context length the workload has on average, not at the length right after the prefill."""
    import torch

    if n_tokens <= 0:
        return
    runner = eng.worker.runner
    bs = runner.cfg.block_size
    g = torch.Generator().manual_seed(seed)
    slots = []
    for req in eng.scheduler.running:
        c = req.num_computed_tokens
        if eng.kv.allocate_slots(req, n_tokens + len(req.spec_token_ids) + 1) is None:
            raise RuntimeError("KV cache too small for the requested decode context")
        slots += runner._slots(req.block_ids, c, n_tokens)
        req.output_token_ids.extend(torch.randint(0, vocab, (n_tokens,), generator=g).tolist())
        req.num_computed_tokens = c + n_tokens
    idx = torch.tensor(slots, dtype=torch.int64, device=runner.device)
    caches = list(runner.kv_caches) + [k[0] for k in runner.drafter_kv]
    width = None
    for c in caches:
        for t in (c if isinstance(c, tuple) else (c,)):
            flat = t.view(-1, t.shape[-1] if t.dim() == 3 else t.shape[-2] * t.shape[-1])
            if width != flat.shape[1]:
                width = flat.shape[1]
                rnd = (torch.randn(idx.numel(), width, device=runner.device) * 0.5).to(t.dtype)
            flat[idx] = rnd
    torch.cuda.synchronize()


def module_breakdown(eng, mc):
    """One extra, untimed decode step run eagerly with CUDA events around the top-level module classes.  Returns
    milliseconds per class and the HBM bytes each class has to stream (its parameters once, plus the KV cache for
    attention), so that the line carries achieved / measured-copy-bandwidth fractions."""
    import torch

    runner = eng.worker.runner
    classes = {"MLAAttention": "attention", "GQAAttention": "attention", "MoELayer": "experts", "SwiGLUMLP": "dense_mlp"}
    spans, depth, hooks, nbytes = [], [0], [], {}

    def pre(mod, _inp):
        if depth[0] == 0:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            mod._bd_start = ev
        depth[0] += 1

    def post(mod, _inp, _out):
        depth[0] -= 1
        if depth[0] == 0:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            spans.append((classes[mod.__class__.__name__], mod._bd_start, ev))

    models = [runner.model] + list(runner.drafters)
    for m in models:
        for mod in m.modules():
            kind = classes.get(mod.__class__.__name__)
            if kind is None:
                continue
            hooks.append(mod.register_forward_pre_hook(pre))
            hooks.append(mod.register_forward_hook(post))
    seen = set()
    for m in models:
        for mod in m.modules():
            kind = classes.get(mod.__class__.__name__)
            if kind is None:
                continue
            for prm in mod.parameters():
                if id(prm) not in seen:
                    seen.add(id(prm))
                    nbytes[kind] = nbytes.get(kind, 0) + prm.numel() * prm.element_size()
    graphs, runner.graphs = runner.graphs, None
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    try:
        eng.step()                     # eager warm-up of this path
        torch.cuda.synchronize()
        spans.clear()
        a.record()
        eng.step()
        b.record()
        torch.cuda.synchronize()
    finally:
        runner.graphs = graphs
        for h in hooks:
            h.remove()
    ms = {}
    for kind, e0, e1 in spans:
        ms[kind] = ms.get(kind, 0.0) + e0.elapsed_time(e1)
    total = a.elapsed_time(b)
    ms["other"] = max(0.0, total - sum(ms.values()))
    ctx = sum(r.num_computed_tokens for r in eng.scheduler.running)
    n_kv = len(runner.kv_caches) + len(runner.drafter_kv)
    nbytes["attention"] = nbytes.get("attention", 0) + ctx * mc.kv_bytes_per_token(2) * n_kv
    return {"eager_step_ms": round(total, 2), "ms": {k: round(v, 2) for k, v in ms.items()},
            "hbm_bytes": {k: int(v) for k, v in nbytes.items()}}


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
    out_len = {"deepseek-v3": 1024, "deepseek-v2-lite": 256, "qwen3-30b-a3b": 512}.get(args.config, 0)
    decode_ctx = args.decode_ctx if args.decode_ctx >= 0 else (in_len + out_len // 2 if not (args.batch or args.input_len) else 0)
    total_steps = args.warmup + args.steps
    extra_steps = 8 + (0 if args.no_breakdown else 2) + (0 if args.no_nccl_arm or world == 1 else 8)
    per_req_tokens = max(in_len, decode_ctx) + tpr * (total_steps + extra_steps + 4) + 8
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

    # ---- move to the context length the timed steps are meant to run at (their middle sits at decode_ctx)
    skip = decode_ctx - in_len - 1 - args.warmup - args.steps // 2 if decode_ctx else 0
    fast_forward(eng, skip, mc.vocab_size, 7 + rank)

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
    try:
        nat.check_status()
    except nat.KernelProtocolError:
        print(f"[rank {rank}] a bounded wait ran out; device ms per timed step: {[round(x, 2) for x in step_dev]}",
              file=sys.stderr, flush=True)
        raise
    ctx_mid = statistics.mean(r.num_computed_tokens for r in eng.scheduler.running) - args.steps / 2

    # ---- untimed extras: per-module breakdown of one eager step; the same steps over the NCCL all-to-all baseline
    breakdown = None if args.no_breakdown else module_breakdown(eng, mc)
    nccl_ms = None
    runner = eng.worker.runner
    if world > 1 and not args.no_nccl_arm and not args.attn_tp and getattr(runner, "ep_ctx", None) is not None:
        runner.force_ep_baseline = True        # every rank sets it, so the agreement stays consistent
        for _ in range(2):
            eng.step()
        torch.cuda.synchronize()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        nccl_ms = e0.elapsed_time(e1) / 4
        runner.force_ep_baseline = False
        tt = torch.tensor([nccl_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        nccl_ms = float(tt[0])
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
                       "ctx_at_timing": round(ctx_mid, 1),
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
        peaks = {"hbm_gbs": 6533.2}
        try:
            peaks.update(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))))
        except Exception:  # noqa: BLE001
            pass
        if breakdown is not None:
            fr = {}
            for k, b in breakdown["hbm_bytes"].items():
                t_ms = breakdown["ms"].get(k)
                if t_ms:
                    fr[k] = round(b / (t_ms * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3)
            breakdown["frac_of_measured_hbm_copy"] = fr
            total_b = sum(breakdown["hbm_bytes"].values())
            breakdown["step_frac_of_measured_hbm_copy"] = round(total_b / (dev_ms / args.steps * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3)
            line["breakdown"] = breakdown
        if nccl_ms is not None:
            line["nccl_all_to_all_arm"] = {"ms_per_step": round(nccl_ms, 3), "steps": 4, "mode": "eager, same engine and batch",
                                           "fused_speedup": round(nccl_ms / (dev_ms / args.steps), 3)}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
