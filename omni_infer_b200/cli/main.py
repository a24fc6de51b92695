"""``omni_cli serve <deployment.yml>`` / ``omni_cli status --config <deployment.yml>`` (reference: omni/cli/main.py:31-108).
``serve`` turns the deployment file into a process plan and runs it on this box (``--dry-run`` prints the plan);
``status`` sends one completion through the proxy."""
from __future__ import annotations

import argparse
import json
import sys
import urllib.request

from .config_transform import plan_to_json, transform_deployment_config, write_inventory
from .launch import Launcher


def status(config: str, timeout: float = 30.0) -> int:
    import yaml
    cfg = yaml.safe_load(open(config))
    px = cfg.get("deployment", {}).get("proxy", {})
    url = f"http://{px.get('ip', '127.0.0.1')}:{px.get('listen_port', 8080)}/v1/completions"
    body = json.dumps({"model": cfg.get("services", {}).get("model_path", "model"), "prompt": "hello", "max_tokens": 8,
                       "temperature": 0}).encode()
    try:
        with urllib.request.urlopen(urllib.request.Request(url, data=body, headers={"Content-Type": "application/json"}),
                                    timeout=timeout) as r:
            print(json.dumps({"status": r.status, "body": json.loads(r.read() or b"{}")}))
            return 0
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"status": "unreachable", "error": str(e)}))
        return 1


def serve_with_ansible(config: str, dry_run: bool = False, inventory: str = "omni_infer_inventory.yml") -> int:
    """The reference's ``serve``: inventory from the deployment file, then the playbook (omni/cli/main.py:31-80)."""
    import os
    import shutil
    import subprocess
    write_inventory(config, inventory)
    playbook = os.path.join(os.path.dirname(os.path.abspath(__file__)), "omni_infer_server.yml")
    cmd = ["ansible-playbook", "-i", inventory, playbook]
    if dry_run or shutil.which("ansible-playbook") is None:
        print(json.dumps({"inventory": inventory, "command": cmd,
                          "note": "dry run" if dry_run else "ansible-playbook is not installed: run the command where it is"}))
        return 0 if dry_run else 1
    return subprocess.call(cmd)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="omni_cli")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve")
    s.add_argument("config")
    s.add_argument("--dry-run", action="store_true")
    s.add_argument("--log-dir", default="./logs")
    s.add_argument("--restart", action="store_true", help="restart a process that exits instead of stopping everything")
    s.add_argument("--ansible", action="store_true",
                   help="several hosts: write the inventory and run the playbook instead of starting local processes")
    st = sub.add_parser("status")
    st.add_argument("--config", required=True)
    iv = sub.add_parser("inventory", help="write the ansible inventory of a deployment file")
    iv.add_argument("config")
    iv.add_argument("-o", "--output", default="omni_infer_inventory.yml")
    a = ap.parse_args(argv)
    if a.cmd == "status":
        return status(a.config)
    if a.cmd == "inventory":
        print(write_inventory(a.config, a.output))
        return 0
    if a.ansible:
        return serve_with_ansible(a.config, a.dry_run)
    plan = transform_deployment_config(a.config)
    if a.dry_run:
        print(plan_to_json(plan))
        return 0
    return Launcher(plan, a.log_dir, a.restart).run_forever()


if __name__ == "__main__":
    sys.exit(main())
