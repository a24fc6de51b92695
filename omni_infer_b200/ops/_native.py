"""ctypes loader for ``libomni_kernels.so`` (the hand-written sm_100a kernels).

The kernels export a plain C ABI that takes raw device pointers and a ``cudaStream_t``; this
module turns tensors into those arguments.  On a machine with a GPU a missing library is an
error (there is no silent PyTorch fallback for CUDA tensors); on CPU-only machines the library
is optional and the fp32 reference implementations in :mod:`omni_infer_b200.ops` are used.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libomni_kernels.so"
_lib = None
_status = {}

c_int = ctypes.c_int
c_float = ctypes.c_float
c_void_p = ctypes.c_void_p
c_int64 = ctypes.c_int64


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


# kernels launched by one call of each entry point (entry points not listed launch one)
_KERNELS_PER_CALL = {"omni_moe_align": 2}


class _CountingLib:
    """Proxy over the CDLL that counts kernel launches issued through it (benchmarks report the count).
    Launches replayed from CUDA graphs are added by the graph runner through :func:`add_launches`."""

    def __init__(self, cdll):
        self._cdll = cdll
        self.launches = 0
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _n=n):
                self.launches += _n
                return _raw(*args)

            self._cache[name] = fn
        return fn


def lib():
    """Load the kernel library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: run `python -m omni_infer_b200.build` "
                "(CUDA tensors never fall back to PyTorch ops)")
        _lib = _CountingLib(ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL))
    return _lib


def launch_count() -> int:
    return _lib.launches if _lib is not None else 0


def add_launches(n: int) -> None:
    if _lib is not None:
        _lib.launches += n


def ptr(t):
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def status_buffer(device=None) -> torch.Tensor:
    """Per-device int32[4] word {code, site, block, detail} that kernels write when a bounded
    wait gives up.  Zero means every launch so far completed its protocol."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        # a plain tensor even when the first caller runs under inference mode: callers reset it in place later
        with torch.inference_mode(False):
            _status[key] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


class KernelProtocolError(RuntimeError):
    """A kernel gave up on a bounded wait (code, site, block, detail)."""


def _site_kernel(site: int) -> str:
    """Which kernel family a wait-site id belongs to (each family numbers its sites in its own decade)."""
    for lo, hi, name in ((1, 9, "weight-major GEMM"), (11, 19, "prefill attention"), (21, 29, "token-major GEMM"),
                         (31, 39, "MLA decode"), (41, 49, "TP collectives"), (200, 299, "EP dispatch/combine")):
        if lo <= site <= hi:
            return name
    return "an unnamed kernel"


def check_status(device=None, reset: bool = True) -> None:
    """Synchronise and raise :class:`KernelProtocolError` if any kernel reported a failed wait."""
    buf = status_buffer(device)
    vals = buf.tolist()
    if vals[0] != 0:
        if reset:
            buf.zero_()
        what = {1: "mbarrier wait gave up", 2: "flag wait gave up", 3: "index out of bounds (access skipped)",
                4: "capacity exceeded"}.get(vals[0], "kernel error")
        extra = ""
        if 31 <= vals[1] <= 39:
            # the MLA decode kernel leaves what each of its warps was waiting for when the first CTA gave up
            rec = (ctypes.c_int * 32)()
            if lib().omni_mla_debug_read(rec) == 0 and rec[0]:
                waits = {w: (rec[8 + w] >> 16, rec[8 + w] & 0xffff) for w in range(12) if rec[8 + w]}
                extra = (f"; first CTA to give up: block=({rec[1]},{rec[2]},{rec[3]}) tiles={rec[4]} kv_len={rec[5]} "
                         f"first_tile={rec[6]} splits={rec[7]} warp waits (site, detail)={waits} "
                         f"odd-phase masks: kv_full={rec[20]:09b} kv_empty={rec[21]:09b} s/p/o={rec[22]:06b}")
        raise KernelProtocolError(f"{what} in {_site_kernel(vals[1])}: code={vals[0]} site={vals[1]} block={vals[2]} "
                                  f"detail={vals[3]}{extra}")


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
