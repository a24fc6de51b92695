"""Function-level, non-intrusive profiling driven by a YAML name list
(reference: omni/adaptors/vllm/patches/profiler_patches/apply_profiler_patches.py:25-155, prof_wrapper.py:15-272).

``PROFILING_NAMELIST=<file.yml>`` lists targets ``module[:Class].function`` with a wrapper type:
  timer      wall time per call, logged (and kept in ``TIMINGS``)
  viztracer  trace the call with VizTracer when it is installed
  torchprof  run the call under torch.profiler (CPU + CUDA), trace written to ``profile_dir``
  marker     call named entry / exit callbacks (the reference executes code snippets; named callbacks from
             ``MARKER_CALLBACKS`` are used here instead), e.g. the per-request timeline logger
NVTX ranges are added around every wrapped call when CUDA is available."""
from __future__ import annotations

import functools
import importlib
import logging
import time
from collections import defaultdict

import torch

logger = logging.getLogger("omni_infer_b200.profiler")
TIMINGS: dict = defaultdict(list)
MARKER_CALLBACKS: dict = {}


def timeline_marker(action: str, role: str = ""):
    """Per-request timeline line ``<<<Action: ...; Timestamp: ...; RequestID: ...; Role: ...`` (the format of the
    reference's omnilogger name list)."""
    def cb(args, kwargs, result=None):
        rid = kwargs.get("request_id") or next((getattr(a, "request_id", None) for a in args if hasattr(a, "request_id")), "")
        logger.info("<<<Action: %s; Timestamp:%.6f; RequestID:%s; Role:%s", action, time.time(), rid, role)
    return cb


def _nvtx_push(name):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)


def _nvtx_pop():
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def timer_wrapper(fn, name):
    @functools.wraps(fn)
    def w(*a, **k):
        _nvtx_push(name)
        t0 = time.perf_counter()
        try:
            return fn(*a, **k)
        finally:
            dt = time.perf_counter() - t0
            _nvtx_pop()
            TIMINGS[name].append(dt)
            logger.info("[timer] %s %.3f ms", name, dt * 1e3)
    return w


def viztracer_wrapper(fn, name, output_dir="."):
    @functools.wraps(fn)
    def w(*a, **k):
        try:
            from viztracer import VizTracer
        except ImportError:
            return fn(*a, **k)
        with VizTracer(output_file=f"{output_dir}/{name.replace('.', '_')}_{time.time_ns()}.json", verbose=0):
            return fn(*a, **k)
    return w


def torchprof_wrapper(fn, name, profile_dir="./profiler_traces"):
    @functools.wraps(fn)
    def w(*a, **k):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        with torch.profiler.profile(activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(profile_dir)):
            return fn(*a, **k)
    return w


def marker_wrapper(fn, name, entry=None, exit=None):
    e_cb = MARKER_CALLBACKS.get(entry) if isinstance(entry, str) else entry
    x_cb = MARKER_CALLBACKS.get(exit) if isinstance(exit, str) else exit

    @functools.wraps(fn)
    def w(*a, **k):
        if e_cb:
            e_cb(a, k)
        r = fn(*a, **k)
        if x_cb:
            x_cb(a, k, r)
        return r
    return w


WRAPPERS = {"timer": timer_wrapper, "viztracer": viztracer_wrapper, "torchprof": torchprof_wrapper,
            "torchnpu": torchprof_wrapper, "marker": marker_wrapper}


def patch_target(target: str, wrapper_type: str = "timer", **opts):
    """target = 'pkg.module:Class.method' or 'pkg.module.function'.  Returns the original callable."""
    if ":" in target:
        mod_name, rest = target.split(":", 1)
        obj = importlib.import_module(mod_name)
        parts = rest.split(".")
    else:
        mod_name, fn_name = target.rsplit(".", 1)
        obj = importlib.import_module(mod_name)
        parts = [fn_name]
    for p in parts[:-1]:
        obj = getattr(obj, p)
    orig = getattr(obj, parts[-1])
    setattr(obj, parts[-1], WRAPPERS[wrapper_type](orig, target, **opts))
    return orig


def apply_patches(namelist_path: str) -> list:
    """YAML: {type: timer, targets: [...]} or a list of {target, type, entry, exit, ...} entries."""
    import yaml

    spec = yaml.safe_load(open(namelist_path)) or {}
    entries = spec if isinstance(spec, list) else [dict(target=t, type=spec.get("type", "timer")) for t in spec.get("targets", [])]
    done = []
    for e in entries:
        e = dict(e)
        target, typ = e.pop("target"), e.pop("type", "timer")
        try:
            patch_target(target, typ, **e)
            done.append(target)
        except (ImportError, AttributeError) as ex:
            logger.warning("cannot patch %s: %s", target, ex)
    return done


def run_model_with_profiling(fn, iters: int = 6, profile_dir: str = "./profiler_traces"):
    """Forward-only profiling helper (PROFILING_FORWARD=1 in the reference): a few iterations under the profiler."""
    out = None
    acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with torch.profiler.profile(activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(profile_dir)):
        for _ in range(iters):
            out = fn()
    return out


class DeviceTimer:
    """CUDA-event timing of a region on the current stream; ``elapsed_ms_max_over_ranks`` reduces over the job."""

    def __enter__(self):
        self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        self.a.record()
        return self

    def __exit__(self, *exc):
        self.b.record()
        torch.cuda.synchronize()
        self.ms = self.a.elapsed_time(self.b)

    def elapsed_ms_max_over_ranks(self) -> float:
        import torch.distributed as dist
        if dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([self.ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return self.ms
