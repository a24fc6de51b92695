"""Launcher of the C++ global proxy (``csrc/proxy``), the counterpart of the reference's ``global_proxy.sh``
(omni/accelerators/sched/global_proxy/README.md:54-62): same option names for the server lists and the balancer
choice, start / stop / status, optional CPU pinning of the workers, a dry run that prints the resolved
configuration, roll-back to the last configuration that started (the reference keeps a copy of the previous
nginx.conf and restores it when the new one does not come up), and the OS tuning the reference applies before
starting (file-descriptor limit for the proxy process; the system-wide sysctl settings are only printed unless
``--apply-os-tuning`` is given, because they outlive the process).

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
    if a.timeline:
        cmd.append("--timeline")
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
    ap.add_argument("--timeline", action="store_true", help="per-request stage lines in the log (utils/timeline.py reads them)")
    ap.add_argument("--pid-file", default="/tmp/omni_proxy.pid")
    ap.add_argument("--log-file", default="/tmp/omni_proxy.log")
    ap.add_argument("--stop", action="store_true")
    ap.add_argument("--status", action="store_true")
    ap.add_argument("--rollback", action="store_true", help="restart with the last configuration that came up")
    ap.add_argument("--state-dir", default="/tmp/omni_proxy_state", help="where the current / previous configuration are kept")
    ap.add_argument("--nofile", type=int, default=65535, help="file-descriptor limit of the proxy process")
    ap.add_argument("--apply-os-tuning", action="store_true", help="also run the system-wide sysctl commands (needs root)")
    ap.add_argument("--dry-run", action="store_true")
    return ap.parse_args(argv)


OS_TUNING = (("net.core.somaxconn", "65535"), ("net.ipv4.tcp_max_syn_backlog", "65535"),
             ("net.ipv4.ip_local_port_range", "1024 65535"), ("net.ipv4.tcp_tw_reuse", "1"),
             ("net.ipv4.tcp_fin_timeout", "15"))


def os_tuning_commands() -> list:
    return [["sysctl", "-w", f"{k}={v}"] for k, v in OS_TUNING]


def _raise_nofile(limit: int):
    def f():
        import resource
        soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
        want = min(limit, hard) if hard != resource.RLIM_INFINITY else limit
        if want > soft:
            resource.setrlimit(resource.RLIMIT_NOFILE, (want, hard))
    return f


def _start(cmd: list, a, cores=None):
    def preexec():
        _raise_nofile(a.nofile)()
        if cores:
            os.sched_setaffinity(0, cores)
    # the proxy outlives this launcher: its own session and its own log file, not the launcher's pipes
    log = open(a.log_file, "ab")
    proc = subprocess.Popen(cmd, preexec_fn=preexec, stdin=subprocess.DEVNULL, stdout=log, stderr=log, start_new_session=True)
    time.sleep(0.3)
    return proc if proc.poll() is None else None


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
    state = Path(a.state_dir)
    cur, prev = state / "current.json", state / "previous.json"
    if a.status:
        try:
            pid = int(Path(a.pid_file).read_text())
            os.kill(pid, 0)
            print(json.dumps({"running": True, "pid": pid, "config": json.loads(cur.read_text()) if cur.exists() else None}))
        except (FileNotFoundError, ProcessLookupError, ValueError):
            print(json.dumps({"running": False}))
        return 0
    cmd = build_command(a)
    if a.rollback:
        if not prev.exists():
            print("no previous configuration to roll back to", file=sys.stderr)
            return 1
        cmd = json.loads(prev.read_text())["command"]
    if a.dry_run:
        out = subprocess.run(cmd + ["--dump-config"], capture_output=True, text=True)
        print(json.dumps({"command": cmd, "resolved": json.loads(out.stdout), "nofile": a.nofile,
                          "os_tuning": [" ".join(c) for c in os_tuning_commands()]}))
        return 0
    if a.apply_os_tuning:
        for c in os_tuning_commands():
            subprocess.run(c, check=False)
    cores = None
    if a.start_core_index >= 0 and hasattr(os, "sched_setaffinity"):
        cores = set(range(a.start_core_index, a.start_core_index + a.core_num))
    state.mkdir(parents=True, exist_ok=True)
    proc = _start(cmd, a, cores)
    if proc is None:
        # the new configuration does not come up: fall back to the one that did, as the reference's launcher does
        print("proxy exited at start-up", file=sys.stderr)
        if cur.exists() and not a.rollback:
            old = json.loads(cur.read_text())["command"]
            proc = _start(old, a, cores)
            if proc is not None:
                Path(a.pid_file).write_text(str(proc.pid))
                print(f"rolled back to the previous configuration, proxy pid {proc.pid}", file=sys.stderr)
        return 1
    if cur.exists() and not a.rollback:
        prev.write_text(cur.read_text())
    cur.write_text(json.dumps({"command": cmd, "started": time.time()}))
    Path(a.pid_file).write_text(str(proc.pid))
    print(f"proxy pid {proc.pid} listening on {a.listen_host}:{a.listen_port}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
