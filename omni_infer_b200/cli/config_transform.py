"""Deployment YAML -> concrete process plan (reference: omni/cli/config_transform.py:123-354 turns the same schema
into an ansible inventory; here the plan is a list of local processes because one NVSwitch box replaces the
cluster of hosts).

Schema (kept from omni/cli/omni_infer_deployment.yml):
  deployment:
    prefill: {group1: [{ip, ascend_rt_visible_devices | devices, master_port, api_port ...}], ...}
    decode:  {group1: [...]}
    proxy:   {ip, listen_port, prefill_lb_sdk, decode_lb_sdk, core_num, start_core_index}
  services:
    model_path, tensor_parallel_size (prefill), max_model_len / max_num_seqs / ... per role, additional_config
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Optional

import yaml


@dataclass
class ProcessSpec:
    name: str
    role: str                     # prefill | decode | proxy
    argv: list
    env: dict = field(default_factory=dict)
    api_port: int = 0
    log_file: str = ""


def _devices(node: dict) -> list:
    d = node.get("devices", node.get("ascend_rt_visible_devices", node.get("cuda_visible_devices", "")))
    if isinstance(d, (list, tuple)):
        return [int(x) for x in d]
    return [int(x) for x in str(d).replace(" ", "").split(",") if x != ""]


def transform_deployment_config(path_or_dict) -> list:
    cfg = yaml.safe_load(open(path_or_dict)) if isinstance(path_or_dict, str) else dict(path_or_dict)
    dep, svc = cfg.get("deployment", {}), cfg.get("services", {})
    model = svc.get("model_path", svc.get("model", "tiny-deepseek-v3"))
    procs: list = []
    endpoints = {"prefill": [], "decode": []}
    control_port = int(svc.get("kv_control_port", 5568))
    for role in ("prefill", "decode"):
        groups = dep.get(role, {}) or {}
        idx = 0
        for gname, nodes in groups.items():
            for node in nodes:
                devs = _devices(node)
                api_port = int(node.get("api_port", node.get("base_api_port", 9000 + (0 if role == "prefill" else 100) + idx)))
                role_svc = dict(svc.get(role, {}))
                kv = {"kv_role": "kv_producer" if role == "prefill" else "kv_consumer",
                      "engine_id": f"{role}-{idx}", "endpoint": f"tcp://{node.get('ip', '127.0.0.1')}:{control_port + len(procs)}",
                      "transport": "tcp"}
                argv = ["-m", "omni_infer_b200.engine.api_server", "--model", str(model), "--port", str(api_port),
                        "--max-model-len", str(role_svc.get("max_model_len", 32000 if role == "prefill" else 16384)),
                        "--max-num-seqs", str(role_svc.get("max_num_seqs", 16 if role == "prefill" else 256)),
                        "--max-num-batched-tokens", str(role_svc.get("max_num_batched_tokens", 30000 if role == "prefill" else 8192)),
                        "--kv-transfer-config", json.dumps(kv)]
                if role_svc.get("additional_config"):
                    argv += ["--additional-config", json.dumps(role_svc["additional_config"])]
                if role == "prefill" and role_svc.get("enforce_eager", True):
                    argv.append("--enforce-eager")
                if role_svc.get("num_speculative_tokens"):
                    argv += ["--num-speculative-tokens", str(role_svc["num_speculative_tokens"])]
                env = {"CUDA_VISIBLE_DEVICES": ",".join(map(str, devs)), "ROLE": role,
                       "MODEL_EXTRA_CFG_PATH": str(role_svc.get("model_extra_cfg_path", ""))}
                procs.append(ProcessSpec(f"{role}-{gname}-{idx}", role, argv, env, api_port, f"server_{role}_{idx}.log"))
                endpoints[role].append(f"{node.get('ip', '127.0.0.1')}:{api_port}")
                idx += 1
    px = dep.get("proxy")
    if px:
        argv = ["-m", "omni_infer_b200.accelerators.sched.global_proxy", "--listen-port", str(px.get("listen_port", 8080)),
                "--decode-servers-list", ",".join(endpoints["decode"]),
                "--prefill-lb-sdk", px.get("prefill_lb_sdk", "pd_score_balance"),
                "--decode-lb-sdk", px.get("decode_lb_sdk", "pd_score_balance"), "--core-num", str(px.get("core_num", 1))]
        if endpoints["prefill"]:
            argv += ["--prefill-servers-list", ",".join(endpoints["prefill"])]
        if px.get("start_core_index") is not None:
            argv += ["--start-core-index", str(px["start_core_index"])]
        procs.append(ProcessSpec("proxy", "proxy", argv, {}, int(px.get("listen_port", 8080)), "proxy.log"))
    return procs


def plan_to_json(procs: list) -> str:
    return json.dumps([asdict(p) for p in procs], indent=1)


# ---------------------------------------------------------------------------------------------------------------
# several hosts: the same deployment file as an ansible inventory (reference: omni/cli/config_transform.py:123-354
# writes omni_infer_inventory.yml with host groups P / D / C and per-host node_rank, kv_rank, ports and devices)
# ---------------------------------------------------------------------------------------------------------------
def plan_to_inventory(path_or_dict, user: str = "root", code_path: str = "/workspace/omni_infer_b200",
                      log_path: str = "/workspace/logs", docker_image: str = "omni-infer-b200:latest") -> dict:
    """Inventory for ``omni_infer_server.yml``: one host entry per prefill / decode instance and one for the proxy.
    ``node_rank`` counts the hosts of a group, ``kv_rank`` the instances of a role; ``argv`` / ``env`` are what the
    local launcher would start, so a host runs exactly the process the single-box plan runs."""
    cfg = yaml.safe_load(open(path_or_dict)) if isinstance(path_or_dict, str) else dict(path_or_dict)
    procs = transform_deployment_config(cfg)
    dep = cfg.get("deployment", {})
    hosts = {"P": {}, "D": {}, "C": {}}
    by_name = {p.name: p for p in procs}
    for role, key in (("prefill", "P"), ("decode", "D")):
        idx = 0
        for gname, nodes in (dep.get(role, {}) or {}).items():
            for node_rank, node in enumerate(nodes):
                spec = by_name[f"{role}-{gname}-{idx}"]
                kv = json.loads(spec.argv[spec.argv.index("--kv-transfer-config") + 1])
                hosts[key][f"{key.lower()}{idx}"] = {
                    "control_port": int(kv["endpoint"].rsplit(":", 1)[1]),      # where this instance's KV control listens
                    "ansible_host": node.get("ip", "127.0.0.1"), "ansible_user": node.get("user", user),
                    "role": role, "group": gname, "node_rank": node_rank, "kv_rank": idx, "api_port": spec.api_port,
                    "devices": spec.env["CUDA_VISIBLE_DEVICES"], "master_port": int(node.get("master_port", 29500 + idx)),
                    "server_argv": spec.argv, "server_env": spec.env, "log_file": spec.log_file,
                }
                idx += 1
    if "proxy" in by_name:
        px = dep["proxy"]
        hosts["C"]["c0"] = {"ansible_host": px.get("ip", "127.0.0.1"), "ansible_user": px.get("user", user), "role": "proxy",
                            "listen_port": by_name["proxy"].api_port, "proxy_argv": by_name["proxy"].argv,
                            "log_file": by_name["proxy"].log_file}
    return {"all": {"vars": {"code_path": code_path, "log_path": log_path, "docker_image": docker_image,
                             "container_name": "omni_infer_b200", "python": "python3"},
                    "children": {k: {"hosts": v} for k, v in hosts.items()}}}


def write_inventory(path_or_dict, out_path: str, **kw) -> str:
    inv = plan_to_inventory(path_or_dict, **kw)
    with open(out_path, "w") as f:
        yaml.safe_dump(inv, f, sort_keys=False)
    return out_path
