#!/usr/bin/env python
"""Prefill/decode-disaggregated serving under Poisson arrivals (scaled form of the 4P + 4D workload).

One prefill engine and one decode engine run in this process on the same GPU and are stepped in turn; a request is
prefilled on the prefill engine, its KV blocks are pushed into the decode engine's paged cache by the push kernel
(the same connector protocol as between processes: push request, acknowledgement, delayed free, prefilled-token
reuse), and it decodes on the decode engine.  Reports TTFT and TPOT percentiles from wall-clock timestamps.  With both
engines time-sharing one GPU the absolute numbers are not those of eight GPUs; the script is the workload definition and
a functional end-to-end run of the PD path on the device.

    python benchmarks/config4_pd_poisson.py --config qwen3-30b-a3b --rate 8 --duration 60 --input-len 4096 --output-len 512
    python benchmarks/config4_pd_poisson.py --config small --rate 20 --duration 5 --input-len 128 --output-len 32   # quick

Reference workflow: omni/accelerators/pd/omni_cache_connector_v1.py, omni/accelerators/sched/global_proxy (two-phase
P -> D request flow)."""
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


def pct(xs, q):
    if not xs:
        return None
    xs = sorted(xs)
    return round(xs[min(len(xs) - 1, int(q * len(xs)))] * 1e3, 2)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="small", choices=["small", "qwen3-30b-a3b"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--rate", type=float, default=8.0, help="requests per second")
    ap.add_argument("--duration", type=float, default=10.0, help="seconds of arrivals")
    ap.add_argument("--input-len", type=int, default=512)
    ap.add_argument("--output-len", type=int, default=64)
    ap.add_argument("--max-decode-batch", type=int, default=128)
    a = ap.parse_args()
    device = "cuda" if torch.cuda.is_available() else "cpu"
    mc = get_config("qwen3-30b-a3b") if a.config == "qwen3-30b-a3b" else get_config("small-deepseek")
    if a.layers:
        mc.num_hidden_layers = a.layers
    bs = 128 if device == "cuda" else 16
    per_req = a.input_len + a.output_len + bs
    n_req = max(1, int(a.rate * a.duration))
    live = min(n_req, a.max_decode_batch + 8)

    def engine(role, name, seqs, blocks):
        import copy
        return EngineCore(EngineConfig(
            model=mc.name, block_size=bs, num_kv_blocks=blocks, max_num_seqs=seqs, max_model_len=per_req + bs,
            max_num_batched_tokens=max(8192, a.input_len), device=device, seed=0, enforce_eager=device == "cpu",
            kv_transfer_config={"kv_role": role, "engine_id": name, "endpoint": f"inproc://{name}", "sync_timeout_s": 20.0,
                                "retries": 3, "retry_wait_s": 0.5}), model_cfg=copy.deepcopy(mc))

    p_blocks = 16 * (a.input_len // bs + 2) + 2
    P = engine("kv_producer", "prefill0", 8, p_blocks)
    d_blocks = live * (per_req // bs + 2) + 2
    d_seqs = a.max_decode_batch
    if device == "cuda":
        # both engines hold the weights; keep the decode cache inside what is left of the device (never size a run so that
        # it can exhaust memory)
        wbytes = sum(q.numel() * q.element_size() for q in P.worker.runner.model.parameters())
        per_block = P.worker.runner.kv_bytes_per_block()
        total = torch.cuda.get_device_properties(0).total_memory
        room = int(total * 0.88) - 2 * wbytes - p_blocks * per_block
        fit = max(0, room // per_block)
        if fit < d_blocks:
            d_seqs = max(1, int((fit - 2) // (per_req // bs + 2)) - 8)
            d_blocks = (d_seqs + 8) * (per_req // bs + 2) + 2
            print(f"decode batch reduced to {d_seqs} sequences to fit the device", file=sys.stderr)
    D = engine("kv_consumer", "decode0", d_seqs, d_blocks)
    g = torch.Generator().manual_seed(0)
    gaps = torch.empty(n_req).exponential_(a.rate, generator=g).tolist()
    arrivals, t = [], 0.0
    for x in gaps:
        t += x
        arrivals.append(t)
    prompts = [torch.randint(0, mc.vocab_size, (a.input_len,), generator=g).tolist() for _ in range(n_req)]
    arrive_t, first_t, last_t, n_tok, tpots = {}, {}, {}, {}, []
    nxt = 0
    t0 = time.perf_counter()
    done = 0
    while done < n_req and time.perf_counter() - t0 < a.duration * 6 + 120:
        now = time.perf_counter() - t0
        while nxt < n_req and arrivals[nxt] <= now:
            rid = f"r{nxt}"
            arrive_t[rid] = arrivals[nxt]
            P.add_request(prompts[nxt], SamplingParams(max_tokens=1), request_id=rid, kv_transfer_params={"do_remote_decode": True})
            nxt += 1
        progressed = False
        if P.scheduler.has_unfinished:
            for out in P.step():
                progressed = True
                if out.finished:
                    rid = out.request_id
                    first_t[rid] = time.perf_counter() - t0           # the prefill instance produced the first token
                    D.add_request(prompts[int(rid[1:])], SamplingParams(max_tokens=a.output_len, ignore_eos=True), request_id=rid,
                                  kv_transfer_params=dict(out.kv_transfer_params))
        else:
            P.step()                                                   # lets the producer see finished transfers
        if D.has_unfinished:
            for out in D.step():
                progressed = True
                rid = out.request_id
                tnow = time.perf_counter() - t0
                k = len(out.new_token_ids)
                if k and rid in last_t:
                    tpots.append((tnow - last_t[rid]) / k)
                if k:
                    last_t[rid] = tnow
                    n_tok[rid] = n_tok.get(rid, 0) + k
                if out.finished:
                    done += 1
        if not progressed:
            time.sleep(0.0005)
    wall = time.perf_counter() - t0
    if device == "cuda":
        torch.cuda.synchronize()
        from omni_infer_b200.ops import _native as nat
        nat.check_status()
    ttft = [first_t[r] - arrive_t[r] for r in first_t]
    print(json.dumps({"config": a.config, "layers": mc.num_hidden_layers, "requests": n_req, "finished": done, "rate_req_s": a.rate,
                      "input_len": a.input_len, "output_len": a.output_len, "wall_s": round(wall, 2),
                      "ttft_ms": {"p50": pct(ttft, 0.5), "p99": pct(ttft, 0.99)},
                      "tpot_ms": {"p50": pct(tpots, 0.5), "p99": pct(tpots, 0.99)},
                      "decode_tok_s": round(sum(n_tok.values()) / wall, 1), "topology": "1 prefill + 1 decode engine on one device"}))


if __name__ == "__main__":
    main()
