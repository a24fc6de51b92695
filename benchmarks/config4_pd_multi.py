#!/usr/bin/env python
"""Prefill/decode-disaggregated serving under Poisson arrivals, one process and one GPU per instance (xPyD, e.g. 4P + 4D
on eight GPUs).

Starts P prefill API servers and D decode API servers (one engine each, GPU i for instance i), the C++ global proxy in
front of them, and a client that sends streaming completion requests to the proxy at Poisson arrival times.  A request
takes the whole production path: proxy -> prefill instance (one token) -> hand-over parameters -> decode instance, whose
connector asks the prefill instance to push the request's KV blocks into its paged cache (CUDA IPC mapping, copy kernel
over NVLink) -> token stream relayed by the proxy.  Reports TTFT (first streamed token at the client) and TPOT
percentiles, request and token throughput, and the proxy's per-stage timeline when ``--timeline`` is given.

    python benchmarks/config4_pd_multi.py --prefill 4 --decode 4 --config qwen3-30b-a3b --rate 8 --duration 60 \
        --input-len 4096 --output-len 512
    python benchmarks/config4_pd_multi.py --prefill 1 --decode 1 --config tiny --device cpu --rate 4 --duration 3 \
        --input-len 48 --output-len 8                                                          # functional check

Reference workflow: tools/scripts/pd_run.sh + global_proxy.sh (one prefill and one decode pod group behind the proxy),
omni/accelerators/pd/omni_cache_connector_v1.py."""
import argparse
import json
import os
import random
import socket
import subprocess
import sys
import threading
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def pct(xs, q):
    if not xs:
        return None
    xs = sorted(xs)
    return round(xs[min(len(xs) - 1, int(q * len(xs)))] * 1e3, 2)


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def wait_health(port, proc, limit_s):
    t0 = time.time()
    while time.time() - t0 < limit_s:
        if proc.poll() is not None:
            return False
        try:
            urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1).read()
            return True
        except Exception:
            time.sleep(0.5)
    return False


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prefill", type=int, default=1)
    ap.add_argument("--decode", type=int, default=1)
    ap.add_argument("--config", default="qwen3-30b-a3b", choices=["tiny", "small", "qwen3-30b-a3b"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--rate", type=float, default=8.0, help="requests per second over the whole deployment")
    ap.add_argument("--duration", type=float, default=60.0, help="seconds of arrivals")
    ap.add_argument("--input-len", type=int, default=4096)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--max-decode-batch", type=int, default=128)
    ap.add_argument("--start-timeout", type=float, default=600.0)
    ap.add_argument("--timeline", action="store_true")
    ap.add_argument("--logdir", default="config4_logs")
    a = ap.parse_args()

    model = {"tiny": "tiny-deepseek-v3", "small": "small-deepseek", "qwen3-30b-a3b": "qwen3-30b-a3b"}[a.config]
    vocab = {"tiny": 1024, "small": 4096, "qwen3-30b-a3b": 151936}[a.config]
    bs = 128 if a.device == "cuda" else 16
    per_req = a.input_len + a.output_len + 2 * bs
    over = {"num_hidden_layers": a.layers} if a.layers else {}
    os.makedirs(a.logdir, exist_ok=True)
    for f in os.listdir(a.logdir):               # timeline files are appended to: start from empty ones
        if f.endswith(".timeline"):
            os.unlink(os.path.join(a.logdir, f))
    procs, logs = [], []
    env0 = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))

    def start_instance(role, idx, gpu):
        port, kv_port = free_port(), free_port()
        name = f"{role}{idx}"
        kv = {"kv_role": "kv_producer" if role == "prefill" else "kv_consumer", "engine_id": name,
              "endpoint": f"tcp://127.0.0.1:{kv_port}", "sync_timeout_s": 30.0, "retries": 3, "retry_wait_s": 2.0}
        seqs = 8 if role == "prefill" else a.max_decode_batch
        cmd = [sys.executable, "-m", "omni_infer_b200.engine.api_server", "--model", model, "--host", "127.0.0.1", "--port", str(port),
               "--max-num-seqs", str(seqs), "--max-model-len", str(per_req), "--block-size", str(bs),
               "--max-num-batched-tokens", str(max(8192, a.input_len)), "--kv-transfer-config", json.dumps(kv)]
        if over:
            cmd += ["--model-overrides", json.dumps(over)]
        if a.device == "cpu":
            cmd += ["--device", "cpu", "--enforce-eager", "--num-kv-blocks", str((seqs + 8) * (per_req // bs + 2) + 2)]
        env = dict(env0)
        if a.device == "cuda":
            env["CUDA_VISIBLE_DEVICES"] = str(gpu)
        if a.timeline:
            env["OMNI_TIMELINE"] = os.path.join(a.logdir, f"{name}.timeline")
        log = open(os.path.join(a.logdir, f"{name}.log"), "w")
        logs.append(log)
        p = subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL)
        procs.append(p)
        return name, port, p

    result = {"config": a.config, "prefill_instances": a.prefill, "decode_instances": a.decode, "rate": a.rate,
              "input_len": a.input_len, "output_len": a.output_len}
    proxy = None
    try:
        t_start = time.time()
        pre = [start_instance("prefill", i, i) for i in range(a.prefill)]
        dec = [start_instance("decode", i, a.prefill + i) for i in range(a.decode)]
        for name, port, p in pre + dec:
            if not wait_health(port, p, a.start_timeout):
                raise RuntimeError(f"instance {name} did not come up (see {a.logdir}/{name}.log)")
        result["start_s"] = round(time.time() - t_start, 1)
        from omni_infer_b200.build import PROXY_BIN, build_proxy
        if not PROXY_BIN.exists():
            build_proxy()
        pport = free_port()
        plog = open(os.path.join(a.logdir, "proxy.log"), "w")
        logs.append(plog)
        pcmd = [str(PROXY_BIN), "--listen", f"127.0.0.1:{pport}", "--prefill-servers", ",".join(f"127.0.0.1:{p}" for _, p, _ in pre),
                "--decode-servers", ",".join(f"127.0.0.1:{p}" for _, p, _ in dec), "--prefill-lb", "pd_score_balance",
                "--decode-lb", "pd_score_balance", "--log-level", "1", "--threads", "256"]
        if a.timeline:
            pcmd.append("--timeline")
        proxy = subprocess.Popen(pcmd, stderr=plog, stdout=plog, stdin=subprocess.DEVNULL)
        procs.append(proxy)
        if not wait_health(pport, proxy, 30):
            raise RuntimeError("the proxy did not come up")

        rng = random.Random(0)
        n_req = max(1, int(a.rate * a.duration))
        arrivals, t = [], 0.0
        for _ in range(n_req):
            t += rng.expovariate(a.rate)
            arrivals.append(t)
        prompts = [[rng.randrange(vocab) for _ in range(a.input_len)] for _ in range(min(n_req, 64))]
        rec = [None] * n_req
        lock = threading.Lock()

        def one(i):
            body = json.dumps({"prompt": prompts[i % len(prompts)], "max_tokens": a.output_len, "stream": True,
                               "ignore_eos": True}).encode()
            req = urllib.request.Request(f"http://127.0.0.1:{pport}/v1/completions", data=body,
                                         headers={"Content-Type": "application/json", "X-Request-Id": f"c4-{i}"})
            t_send = time.perf_counter()
            first = last = None
            n_out = 0
            try:
                with urllib.request.urlopen(req, timeout=600) as r:
                    for line in r:
                        if not line.startswith(b"data: {"):
                            continue
                        now = time.perf_counter()
                        obj = json.loads(line[6:])
                        k = int(obj.get("output_num_token", 0))
                        if k > n_out:
                            if first is None:
                                first = now
                            last, n_out = now, k
                ok = n_out >= a.output_len
            except Exception as e:      # a failed request is a result, not a crash of the benchmark
                ok = False
                with lock:
                    result.setdefault("errors", []).append(f"{type(e).__name__}: {e}"[:200])
            with lock:
                rec[i] = (ok, t_send, first, last, n_out)

        threads = []
        t0 = time.perf_counter()
        for i, at in enumerate(arrivals):
            delay = t0 + at - time.perf_counter()
            if delay > 0:
                time.sleep(delay)
            th = threading.Thread(target=one, args=(i,), daemon=True)
            th.start()
            threads.append(th)
        deadline = time.perf_counter() + a.duration * 4 + 300
        for th in threads:
            th.join(max(0.0, deadline - time.perf_counter()))
        t_total = time.perf_counter() - t0
        done = [r for r in rec if r and r[0]]
        ttft = [r[2] - r[1] for r in done if r[2]]
        tpot = [(r[3] - r[2]) / (r[4] - 1) for r in done if r[4] > 1]
        result.update({"requests": n_req, "finished": len(done), "wall_s": round(t_total, 2),
                       "ttft_ms": {"p50": pct(ttft, 0.5), "p90": pct(ttft, 0.9), "p99": pct(ttft, 0.99)},
                       "tpot_ms": {"p50": pct(tpot, 0.5), "p90": pct(tpot, 0.9), "p99": pct(tpot, 0.99)},
                       "output_tok_s": round(sum(r[4] for r in done) / t_total, 1),
                       "input_tok_s": round(len(done) * a.input_len / t_total, 1)})
        try:
            m = urllib.request.urlopen(f"http://127.0.0.1:{pport}/metrics", timeout=5).read().decode()
            result["proxy_served"] = {l.split(" ")[0]: int(float(l.split(" ")[1])) for l in m.splitlines() if l.startswith("omni_proxy_served_total")}
        except Exception:
            pass
        # how many requests took the KV hand-over (and not the local-prefill fallback) on the decode side
        pulls = fallbacks = 0
        for name, _, _ in dec:
            f = os.path.join(a.logdir, f"{name}.timeline")
            if a.timeline and os.path.exists(f):
                txt = open(f).read()
                pulls += txt.count("Finish to pull kv")
                fallbacks += txt.count("KV transfer failed")
        if a.timeline:
            result["kv_pulls"], result["local_prefill_fallbacks"] = pulls, fallbacks
            from omni_infer_b200.utils import timeline
            files = [os.path.join(a.logdir, "proxy.log")] + [os.path.join(a.logdir, f"{n}.timeline") for n, _, _ in pre + dec]
            s = timeline.summary(timeline.parse([f for f in files if os.path.exists(f)]))
            top = sorted(s["stages"].items(), key=lambda kv: -kv[1]["p50_ms"])[:8]
            result["timeline_p50_ms"] = {k: round(v["p50_ms"], 2) for k, v in top}
    finally:
        for p in procs:
            if p.poll() is None:
                p.terminate()
        for p in procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.kill()
        for f in logs:
            f.close()
    print(json.dumps(result))
    return 0 if result.get("finished") else 1


if __name__ == "__main__":
    sys.exit(main())
