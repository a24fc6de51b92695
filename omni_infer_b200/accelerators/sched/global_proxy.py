"""Launcher of the C++ global proxy (``csrc/proxy``), the counterpart of the reference's ``global_proxy.sh``
(omni/accelerators/sched/global_proxy/README.md:54-62): same option names for the server lists and the balancer
choice, start / stop / status, optional CPU pinning of the workers, and a dry run that prints the resolved
configuration.

    python -m omni_infer_b200.accelerators.sched.global_proxy --listen-port 8080 \
        --prefill-servers-list 10.0.0.1:9000,10.0.0.2:9000 --decode-servers-list 10.0.0.3:9100 \
        --prefill-lb-sdk pd_score_balance --decode-lb-sdk pd_score_balance
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

POLICIES = ("pd_score_balance", "prefill_score_balance", "weighted_least_active", "length_balance", "greedy_timeout",
            "auto_balance_controller", "least_total_load", "round_robin")


def proxy_binary() -> Path:
    from ...build import PROXY_BIN, build_proxy
    if not PROXY_BIN.exists():
        build_proxy()
    return PROXY_BIN


def build_command(a) -> list:
    cmd = [str(proxy_binary()), "--listen", f"{a.listen_host}:{a.listen_port}", "--decode-servers", a.decode_servers_list,
           "--prefill-lb", a.prefill_lb_sdk, "--decode-lb", a.decode_lb_sdk, "--workers", str(a.core_num),
           "--threads", str(a.threads), "--log-level", str(a.log_level), "--fail-timeout", str(a.fail_timeout),
           "--batch-size", str(a.batch_size), "--decode-req-limit", str(a.decode_req_limit)]
    if a.prefill_servers_list:
        cmd += ["--prefill-servers", a.prefill_servers_list]
    return cmd


def parse(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--listen-host", default="0.0.0.0")
    ap.add_argument("--listen-port", type=int, default=8080)
    ap.add_argument("--prefill-servers-list", default="")
    ap.add_argument("--decode-servers-list", required=True)
    ap.add_argument("--prefill-lb-sdk", default="pd_score_balance", choices=POLICIES)
    ap.add_argument("--decode-lb-sdk", default="pd_score_balance", choices=POLICIES)
    ap.add_argument("--core-num", type=int, default=1, help="worker processes")
    ap.add_argument("--start-core-index", type=int, default=-1, help="pin workers to cores starting here")
    ap.add_argument("--threads", type=int, default=64)
    ap.add_argument("--batch-size", type=int, default=25)
    ap.add_argument("--decode-req-limit", type=int, default=0)
    ap.add_argument("--fail-timeout", type=float, default=10.0)
    ap.add_argument("--log-level", type=int, default=1)
    ap.add_argument("--pid-file", default="/tmp/omni_proxy.pid")
    ap.add_argument("--stop", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    a = parse(argv)
    if a.stop:
        try:
            pid = int(Path(a.pid_file).read_text())
            os.kill(pid, signal.SIGTERM)
            Path(a.pid_file).unlink()
            print(f"stopped proxy pid {pid}")
        except (FileNotFoundError, ProcessLookupError, ValueError):
            print("no running proxy")
        return 0
    cmd = build_command(a)
    if a.dry_run:
        out = subprocess.run(cmd + ["--dump-config"], capture_output=True, text=True)
        print(json.dumps({"command": cmd, "resolved": json.loads(out.stdout)}))
        return 0
    if a.start_core_index >= 0 and hasattr(os, "sched_setaffinity"):
        cores = set(range(a.start_core_index, a.start_core_index + a.core_num))
        preexec = lambda: os.sched_setaffinity(0, cores)  # noqa: E731
    else:
        preexec = None
    proc = subprocess.Popen(cmd, preexec_fn=preexec)
    Path(a.pid_file).write_text(str(proc.pid))
    time.sleep(0.3)
    if proc.poll() is not None:
        print("proxy exited at start-up", file=sys.stderr)
        return 1
    print(f"proxy pid {proc.pid} listening on {a.listen_host}:{a.listen_port}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
