"""One-click single-node launcher for the Qwen models (reference: tools/scripts/run_model_qwen.py:96-526): either a
``mixed`` deployment (every selected GPU runs an engine that prefills and decodes) or ``pd_separate`` (1 prefill
instance + 1 decode instance with the KV cache pushed between them), in both cases fronted by the global proxy.

    python -m omni_infer_b200.cli.run_model_qwen --model-path qwen3-30b-a3b --deploy-mode pd_separate \
        --server-list 0,1,2,3 --service-port 6660 [--graph-true true] [--dry-run]
"""
from __future__ import annotations

import argparse
import json
import sys

from .config_transform import ProcessSpec, plan_to_json
from .launch import Launcher, dp_rank_env


def parse(argv=None):
    ap = argparse.ArgumentParser(prog="run_model_qwen", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-path", required=True)
    ap.add_argument("--deploy-mode", default="default", choices=["default", "mixed", "pd_separate"])
    ap.add_argument("--graph-true", default="false", help="'true' = CUDA-graph decode, 'false' = eager")
    ap.add_argument("--network-interface", default=None, help="accepted for compatibility; one box needs none")
    ap.add_argument("--host-ip", default="127.0.0.1")
    ap.add_argument("--model-name", default="default_model")
    ap.add_argument("--log-path", default="./apiserverlog")
    ap.add_argument("--server-list", default="0,1,2,3,4,5,6,7", help="GPUs to use")
    ap.add_argument("--service-port", default="6660", help="first API port; pd_separate: 'prefill_port,decode_port'")
    ap.add_argument("--master-port", default="8888")
    ap.add_argument("--https-port", default="8001", help="port the proxy listens on")
    ap.add_argument("--additional-config", default=None)
    ap.add_argument("--max-model-len", type=int, default=32768)
    ap.add_argument("--dry-run", action="store_true")
    return ap.parse_args(argv)


def build_plan(a) -> list:
    gpus = [g for g in a.server_list.replace(" ", "").split(",") if g != ""]
    ports = [int(p) for p in a.service_port.split(",")]
    master = int(a.master_port.split(",")[0])
    eager = a.graph_true.lower() != "true"
    base = ["-m", "omni_infer_b200.engine.api_server", "--model", a.model_path, "--max-model-len", str(a.max_model_len)]
    if a.additional_config:
        base += ["--additional-config", a.additional_config]
    procs, prefill_eps, decode_eps = [], [], []
    if a.deploy_mode in ("default", "mixed"):
        for i, g in enumerate(gpus):
            env = dp_rank_env(i, len(gpus), a.host_ip, master)
            env["CUDA_VISIBLE_DEVICES"] = g
            argv = base + ["--port", str(ports[0] + i), "--data-parallel-rank", str(i)] + (["--enforce-eager"] if eager else [])
            procs.append(ProcessSpec(f"mixed-{i}", "mixed", argv, env, ports[0] + i, f"server_{i}.log"))
            decode_eps.append(f"{a.host_ip}:{ports[0] + i}")
    else:
        half = max(1, len(gpus) // 2)
        groups = {"prefill": gpus[:half], "decode": gpus[half:] or gpus[:half]}
        p_port, d_port = ports[0], (ports[1] if len(ports) > 1 else ports[0] + 100)
        for role, first_port, kv_role, eps in (("prefill", p_port, "kv_producer", prefill_eps), ("decode", d_port, "kv_consumer", decode_eps)):
            gl = groups[role]
            for i, g in enumerate(gl):
                env = dp_rank_env(i, len(gl), a.host_ip, master + (0 if role == "prefill" else 1))
                env.update({"CUDA_VISIBLE_DEVICES": g, "ROLE": role})
                kv = {"kv_connector": "B200PeerPushConnectorV1", "kv_role": kv_role, "engine_id": f"{role}-{i}",
                      "transport": "tcp", "endpoint": f"tcp://{a.host_ip}:{5568 + len(procs)}"}
                argv = base + ["--port", str(first_port + i), "--data-parallel-rank", str(i), "--kv-transfer-config", json.dumps(kv)]
                if role == "prefill" or eager:
                    argv.append("--enforce-eager")
                procs.append(ProcessSpec(f"{role}-{i}", role, argv, env, first_port + i, f"server_{role}_{i}.log"))
                eps.append(f"{a.host_ip}:{first_port + i}")
    px = ["-m", "omni_infer_b200.accelerators.sched.global_proxy", "--listen-port", a.https_port,
          "--decode-servers-list", ",".join(decode_eps)]
    if prefill_eps:
        px += ["--prefill-servers-list", ",".join(prefill_eps)]
    procs.append(ProcessSpec("proxy", "proxy", px, {}, int(a.https_port), "proxy.log"))
    return procs


def main(argv=None) -> int:
    a = parse(argv)
    plan = build_plan(a)
    if a.dry_run:
        print(plan_to_json(plan))
        return 0
    return Launcher(plan, a.log_path).run_forever()


if __name__ == "__main__":
    sys.exit(main())
