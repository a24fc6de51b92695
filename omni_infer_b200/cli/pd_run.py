"""``omni_pd_run``: start the API servers of one prefill or decode instance, with the option names of the
reference's ``pd_run.sh`` (tools/scripts/pd_run.sh:58-104) and the per-rank fan-out of its
``start_api_servers.py`` (tools/scripts/start_api_servers.py:64-194): one API server + engine per data-parallel
rank, each with ``VLLM_DP_SIZE / VLLM_DP_RANK / VLLM_DP_RANK_LOCAL / VLLM_DP_MASTER_IP / VLLM_DP_MASTER_PORT`` in its
environment, free-port probing from ``--base-api-port``, one log file per server, a liveness loop that stops
everything when one server dies, SIGINT clean-up.

Options that only make sense on the reference's hardware (rank tables, HCCL switches, device lists of another
vendor) are accepted and ignored with a warning, so existing launch lines keep working.  ``--dry-run`` prints the
plan as JSON instead of starting anything."""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys

from .config_transform import ProcessSpec, plan_to_json
from .launch import Launcher, dp_rank_env, port_free

logger = logging.getLogger("omni_infer_b200.pd_run")

IGNORED = ("hcc_intra_roce_enable", "hcc_intra_pcie_enable", "hccl_op_expansion_mode", "hccl_buffsize", "kv_buffer_device",
           "vllm_use_v1", "vllm_worker_multiproc_method", "local_decode_server_ip_list", "global_decode_server_ip_list",
           "enable_expert_parallel", "head", "num_gpus")
# options of the reference's script that have a counterpart here: option -> environment variable of the servers
MAPPED = {"gloo_socket_ifname": "GLOO_SOCKET_IFNAME", "tp_socket_ifname": "NCCL_SOCKET_IFNAME",
          "global_rank_table_path": "OMNI_TOPOLOGY", "rank_table_path": "OMNI_LOCAL_TOPOLOGY"}


def parse(argv=None):
    ap = argparse.ArgumentParser(prog="omni_pd_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    # topology / role
    ap.add_argument("--role", default="prefill", choices=["prefill", "decode", "mixed"])
    ap.add_argument("--prefill-pod-num", type=int, default=1)
    ap.add_argument("--decode-pod-num", type=int, default=1)
    ap.add_argument("--vllm-llmdatadist-zmq-port", "--kv-control-port", dest="kv_control_port", default="5568")
    ap.add_argument("--ascend-rt-visible-devices", "--cuda-visible-devices", dest="devices", default="")
    # mock model
    ap.add_argument("--random-mode", type=int, default=0)
    ap.add_argument("--kv-cache-mod", type=int, default=0)
    ap.add_argument("--forward-time", type=int, default=0)
    # multi API server
    ap.add_argument("--num-servers", type=int, default=1)
    ap.add_argument("--num-dp", type=int, default=None)
    ap.add_argument("--server-offset", type=int, default=0)
    ap.add_argument("--master-ip", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=8503)
    ap.add_argument("--base-api-port", type=int, default=9001)
    ap.add_argument("--max-port-attempts", type=int, default=20)
    # engine
    ap.add_argument("--vllm-logging-level", default="INFO")
    ap.add_argument("--model-path", default="tiny-deepseek-v3")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--served-model-name", default="deepseek")
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=None)
    ap.add_argument("--max-num-batched-tokens", type=int, default=None)
    ap.add_argument("--block-size", type=int, default=128)
    ap.add_argument("--log-dir", default="apiserverlog")
    ap.add_argument("--enable-mtp", action="store_true")
    ap.add_argument("--num-speculative-tokens", type=int, default=1)
    # PD separation
    ap.add_argument("--kv-connector", default="B200PeerPushConnectorV1")
    ap.add_argument("--kv-role", default=None, choices=[None, "kv_producer", "kv_consumer", "kv_both"])
    ap.add_argument("--kv-rank", type=int, default=0)
    ap.add_argument("--kv-engine-id", default="0")
    ap.add_argument("--kv-parallel-size", type=int, default=2)
    ap.add_argument("--model-extra-cfg-path", default=os.environ.get("MODEL_EXTRA_CFG_PATH", ""))
    ap.add_argument("--gpu-util", type=float, default=0.9)
    ap.add_argument("--extra-args", default="")
    ap.add_argument("--additional-config", "--additional-args", dest="additional_config", default="")
    ap.add_argument("--vllm-enable-mc2", type=int, default=1, help="fused NVLink dispatch/combine on decode (role of VLLM_ENABLE_MC2)")
    for name in IGNORED + tuple(MAPPED):
        ap.add_argument("--" + name.replace("_", "-"), default=None, nargs="?", const="1", help=argparse.SUPPRESS)
    ap.add_argument("--address", default=None,
                    help="host:port of the first node of an instance that spans several nodes (the reference passes its Ray "
                         "head address here); becomes the rendezvous address of the ranks")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    if a.address:
        host, _, port = a.address.partition(":")
        a.master_ip = host or a.master_ip
        if port.isdigit():
            a.master_port = int(port)
    return a


def build_plan(a) -> list:
    for name in IGNORED:
        if getattr(a, name) is not None:
            logger.warning("--%s is specific to the reference's hardware and has no effect here", name.replace("_", "-"))
    num_dp = a.num_dp if a.num_dp is not None else a.num_servers
    if num_dp < a.num_servers:
        raise ValueError("--num-dp must be at least --num-servers")
    kv_role = a.kv_role or {"prefill": "kv_producer", "decode": "kv_consumer", "mixed": None}[a.role]
    devices = [d for d in str(a.devices).replace(" ", "").split(",") if d != ""]
    procs, port = [], a.base_api_port
    for i in range(a.num_servers):
        rank = a.server_offset + i
        tries = 0
        while not port_free(port) and tries < a.max_port_attempts:
            port += 1
            tries += 1
        argv = ["-m", "omni_infer_b200.engine.api_server", "--model", a.model_path, "--port", str(port),
                "--max-model-len", str(a.max_model_len), "--block-size", str(a.block_size),
                "--tensor-parallel-size", str(a.tp), "--data-parallel-rank", str(rank)]
        if a.max_num_seqs:
            argv += ["--max-num-seqs", str(a.max_num_seqs)]
        if a.max_num_batched_tokens:
            argv += ["--max-num-batched-tokens", str(a.max_num_batched_tokens)]
        if a.enable_mtp:
            argv += ["--num-speculative-tokens", str(a.num_speculative_tokens)]
        if kv_role:
            kv = {"kv_connector": a.kv_connector, "kv_role": kv_role, "kv_rank": a.kv_rank, "kv_parallel_size": a.kv_parallel_size,
                  "engine_id": f"{a.role}-{a.kv_engine_id}-{rank}", "transport": "tcp",
                  "endpoint": f"tcp://{a.master_ip}:{int(a.kv_control_port) + rank}"}
            argv += ["--kv-transfer-config", json.dumps(kv)]
        if a.additional_config:
            argv += ["--additional-config", a.additional_config]
        if a.role == "prefill":
            argv.append("--enforce-eager")
        argv += [x for x in a.extra_args.split() if x]
        env = dp_rank_env(rank, num_dp, a.master_ip, a.master_port)
        env.update({"ROLE": a.role, "PREFILL_POD_NUM": str(a.prefill_pod_num), "DECODE_POD_NUM": str(a.decode_pod_num),
                    "MODEL_EXTRA_CFG_PATH": a.model_extra_cfg_path, "OMNI_USE_FUSED_EP": str(a.vllm_enable_mc2),
                    "OMNI_KV_CONTROL_PORT": str(a.kv_control_port), "VLLM_LOGGING_LEVEL": a.vllm_logging_level,
                    "SERVED_MODEL_NAME": a.served_model_name, "GPU_UTIL": str(a.gpu_util)})
        for name, var in MAPPED.items():
            if getattr(a, name) is not None:
                env[var] = str(getattr(a, name))
        if devices:
            per = max(1, len(devices) // a.num_servers)
            env["CUDA_VISIBLE_DEVICES"] = ",".join(devices[i * per:(i + 1) * per] or devices[-per:])
        if a.random_mode:
            env.update({"RANDOM_MODE": "1", "FORWARD_TIME": str(a.forward_time)})
        if a.kv_cache_mod:
            env.update({"KV_CACHE_MODE": "1", "PREFILL_PROCESS": "1" if a.role == "prefill" else "0"})
        procs.append(ProcessSpec(f"{a.role}-server-{rank}", a.role, argv, env, port, f"server_{rank}.log"))
        port += 1
    return procs


def main(argv=None) -> int:
    a = parse(argv)
    plan = build_plan(a)
    if a.dry_run:
        print(plan_to_json(plan))
        return 0
    return Launcher(plan, a.log_dir).run_forever()


if __name__ == "__main__":
    sys.exit(main())
