"""Local process launcher: starts the processes of a plan (API servers, proxy), one log file each, watches them
and tears everything down when one dies or on SIGINT (reference: tools/scripts/start_api_servers.py:64-305 and
pd_run.sh; one API server + engine per data-parallel rank, env VLLM_DP_* per process)."""
from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
import time


def port_free(port: int, host: str = "127.0.0.1") -> bool:
    with socket.socket() as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host, port))
            return True
        except OSError:
            return False


def dp_rank_env(rank: int, size: int, master_ip: str = "127.0.0.1", master_port: int = 29555) -> dict:
    return {"VLLM_DP_SIZE": str(size), "VLLM_DP_RANK": str(rank), "VLLM_DP_RANK_LOCAL": str(rank),
            "VLLM_DP_MASTER_IP": master_ip, "VLLM_DP_MASTER_PORT": str(master_port),
            "RANK": str(rank), "WORLD_SIZE": str(size), "LOCAL_RANK": str(rank), "MASTER_ADDR": master_ip,
            "MASTER_PORT": str(master_port)}


class Launcher:
    def __init__(self, procs: list, log_dir: str = "./logs", restart: bool = False):
        self.specs, self.log_dir, self.restart = procs, log_dir, restart
        self.children: dict = {}
        os.makedirs(log_dir, exist_ok=True)

    def start(self) -> None:
        for spec in self.specs:
            if spec.api_port and not port_free(spec.api_port):
                raise RuntimeError(f"port {spec.api_port} for {spec.name} is in use")
            self._spawn(spec)

    def _spawn(self, spec) -> None:
        log = open(os.path.join(self.log_dir, spec.log_file or f"{spec.name}.log"), "ab")
        env = dict(os.environ, **{k: v for k, v in spec.env.items() if v != ""})
        self.children[spec.name] = (spec, subprocess.Popen([sys.executable, *spec.argv], env=env, stdout=log, stderr=log))

    def poll(self) -> list:
        """Names of children that exited since the last call (restarted when the policy says so)."""
        dead = []
        for name, (spec, p) in list(self.children.items()):
            if p.poll() is not None:
                dead.append(name)
                if self.restart:
                    self._spawn(spec)
                else:
                    del self.children[name]
        return dead

    def stop(self) -> None:
        for _, p in self.children.values():
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        t0 = time.time()
        for _, p in self.children.values():
            try:
                p.wait(timeout=max(0.1, 10 - (time.time() - t0)))
            except subprocess.TimeoutExpired:
                p.kill()
        self.children.clear()

    def run_forever(self) -> int:
        self.start()
        signal.signal(signal.SIGINT, lambda *a: (_ for _ in ()).throw(KeyboardInterrupt()))
        try:
            while self.children:
                time.sleep(1.0)
                dead = self.poll()
                if dead and not self.restart:
                    print(f"{dead} exited; stopping the deployment", file=sys.stderr)
                    return 1
        except KeyboardInterrupt:
            pass
        finally:
            self.stop()
        return 0
