"""Per-request timeline across the proxy, the prefill engine and the decode engine.

Every process writes one line per request stage,

    <<<Action: Prefill scheduled; Timestamp:1732540000.123456; RequestID:cmpl-1; Role:prefill

(the line format of the reference's omnilogger name list, omni/adaptors/vllm/patches/profiler_patches/assets/
omnilogger_namelist.yml; the reference injects the lines with function patches, here the engine, the API server and
the C++ proxy write them themselves when the timeline is switched on).  The request id is the ``X-Request-Id`` header
that the proxy sets and both engines reuse, so the lines of the three processes join on it.

Writing:   ``OMNI_TIMELINE=<file>`` (or ``stderr``) switches the engine side on; ``OMNI_TIMELINE_ROLE`` names the
           process (``prefill`` / ``decode`` / ``mixed``).  The proxy takes ``--timeline`` and writes to its log.
Reading:   ``python -m omni_infer_b200.utils.timeline proxy.log prefill.log decode.log [--json out.json]`` merges
           the files, prints the stages of every request with the time since the previous one, and the p50 / p90 /
           p99 of each stage-to-stage interval over all requests (the TTFT and TPOT breakdown).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import threading
import time
from collections import defaultdict

LINE = re.compile(r"<<<Action: (?P<action>.*?); Timestamp:\s*(?P<ts>[0-9.]+); RequestID:\s*(?P<rid>[^;]*); Role:\s*(?P<role>\S*)")

_lock = threading.Lock()
_sink = None          # file object, or None when the timeline is off
_role = ""
_configured = False


def configure(path: str | None = None, role: str | None = None) -> bool:
    """Open the sink.  Without arguments the environment decides; returns whether the timeline is on."""
    global _sink, _role, _configured
    with _lock:
        path = path if path is not None else os.environ.get("OMNI_TIMELINE", "")
        _role = role if role is not None else os.environ.get("OMNI_TIMELINE_ROLE", _role or "engine")
        if _sink not in (None, sys.stderr):
            _sink.close()
        _sink = None
        if path:
            _sink = sys.stderr if path == "stderr" else open(path, "a", buffering=1)
        _configured = True
        return _sink is not None


def enabled() -> bool:
    if not _configured:
        configure()
    return _sink is not None


def emit(action: str, request_id: str, role: str | None = None, ts: float | None = None) -> None:
    if not enabled():
        return
    line = f"<<<Action: {action}; Timestamp:{ts if ts is not None else time.time():.6f}; RequestID:{request_id}; Role:{role or _role}\n"
    with _lock:
        if _sink is not None:
            _sink.write(line)


# ------------------------------------------------------------------------------------------------ reading
def parse(paths) -> dict:
    """request id -> list of (timestamp, role, action), sorted by time."""
    out = defaultdict(list)
    for p in paths:
        with open(p, errors="replace") as f:
            for line in f:
                m = LINE.search(line)
                if m and m["rid"].strip():
                    out[m["rid"].strip()].append((float(m["ts"]), m["role"], m["action"].strip()))
    for v in out.values():
        v.sort(key=lambda e: e[0])
    return dict(out)


def _pct(xs, q):
    xs = sorted(xs)
    if not xs:
        return float("nan")
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


def intervals(timelines: dict) -> dict:
    """"role:action -> role:action" -> list of milliseconds between consecutive stages, over all requests."""
    out = defaultdict(list)
    for ev in timelines.values():
        for (t0, r0, a0), (t1, r1, a1) in zip(ev, ev[1:]):
            out[f"{r0}:{a0} -> {r1}:{a1}"].append((t1 - t0) * 1e3)
    return dict(out)


def summary(timelines: dict) -> dict:
    iv = intervals(timelines)
    stages = {k: {"n": len(v), "p50_ms": _pct(v, 0.5), "p90_ms": _pct(v, 0.9), "p99_ms": _pct(v, 0.99)} for k, v in iv.items()}
    total = [(ev[-1][0] - ev[0][0]) * 1e3 for ev in timelines.values() if len(ev) > 1]
    return {"requests": len(timelines), "stages": stages,
            "end_to_end_ms": {"p50": _pct(total, 0.5), "p90": _pct(total, 0.9), "p99": _pct(total, 0.99)}}


def render(timelines: dict, limit: int = 20) -> str:
    lines = []
    for rid, ev in list(timelines.items())[:limit]:
        lines.append(f"request {rid}")
        t_first, prev = ev[0][0], ev[0][0]
        for ts, role, action in ev:
            lines.append(f"  {1e3 * (ts - t_first):10.3f} ms  (+{1e3 * (ts - prev):9.3f})  {role:8s} {action}")
            prev = ts
    s = summary(timelines)
    lines.append(f"{s['requests']} requests; end to end p50 {s['end_to_end_ms']['p50']:.3f} ms, p99 {s['end_to_end_ms']['p99']:.3f} ms")
    for k, v in sorted(s["stages"].items(), key=lambda kv: -kv[1]["p50_ms"]):
        lines.append(f"  {v['p50_ms']:10.3f} ms p50 {v['p99_ms']:10.3f} ms p99  n={v['n']:<5d} {k}")
    return "\n".join(lines) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--json", default="", help="also write the summary here")
    ap.add_argument("--limit", type=int, default=20, help="requests to print in full")
    a = ap.parse_args(argv)
    tl = parse(a.logs)
    sys.stdout.write(render(tl, a.limit))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(summary(tl), f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
