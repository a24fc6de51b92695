"""In-tree native build: CUDA kernels for sm_100a, the placement core and the proxy.

Everything is compiled with explicit ``nvcc``/``g++`` command lines into ``omni_infer_b200/_lib``
so the shared objects travel with the source tree.  ``build_all()`` is incremental: an output is
rebuilt only when one of its inputs is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "_lib"
OBJ_DIR = LIB_DIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]

KERNEL_LIB = LIB_DIR / "libomni_kernels.so"
PLACEMENT_LIB = LIB_DIR / "libomni_placement.so"
PROXY_BIN = LIB_DIR / "omni_proxy"


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return exe


def _newer(inputs, output: Path) -> bool:
    if not output.exists():
        return True
    t = output.stat().st_mtime
    return any(Path(i).stat().st_mtime > t for i in inputs)


def _run(cmd, log: Path | None = None) -> None:
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if log is not None:
        log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("build command failed: " + " ".join(str(c) for c in cmd))


def build_kernels(verbose: bool = False) -> Path:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a and link ``libomni_kernels.so``."""
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    headers = sorted((CSRC / "include").glob("*"))
    sources = sorted((CSRC / "kernels").glob("*.cu"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        if _newer([src, *headers], obj):
            jobs.append(([nvcc, *NVCC_FLAGS, "-I", CSRC / "include", "-c", src, "-o", obj],
                         OBJ_DIR / (src.stem + ".ptxas.log")))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    if jobs or _newer(objs, KERNEL_LIB):
        _run([nvcc, "-shared", "-o", KERNEL_LIB, *objs])
    if verbose:
        print(f"built {KERNEL_LIB} from {len(sources)} sources ({len(jobs)} recompiled)")
    return KERNEL_LIB


def build_placement(verbose: bool = False) -> Path | None:
    """Build the C++ placement core (no CUDA dependency; device copies go through callbacks)."""
    src_dir = CSRC / "placement"
    sources = sorted(src_dir.glob("*.cpp"))
    if not sources:
        return None
    LIB_DIR.mkdir(exist_ok=True)
    headers = sorted(src_dir.glob("*.h"))
    if _newer([*sources, *headers], PLACEMENT_LIB):
        _run(["g++", *CXX_FLAGS, "-shared", "-I", src_dir, "-o", PLACEMENT_LIB,
              *[s for s in sources if not s.name.startswith("test_")]])
    if verbose:
        print(f"built {PLACEMENT_LIB}")
    return PLACEMENT_LIB


def build_proxy(verbose: bool = False) -> Path | None:
    """Build the C++ global proxy (epoll HTTP reverse proxy with the xPyD load balancers)."""
    src_dir = CSRC / "proxy"
    sources = sorted(s for s in src_dir.glob("*.cpp") if not s.name.startswith("test_"))
    if not sources:
        return None
    LIB_DIR.mkdir(exist_ok=True)
    headers = sorted(src_dir.glob("*.h"))
    if _newer([*sources, *headers], PROXY_BIN):
        _run(["g++", *CXX_FLAGS, "-I", src_dir, "-o", PROXY_BIN, *sources])
    if verbose:
        print(f"built {PROXY_BIN}")
    return PROXY_BIN


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose)
    build_placement(verbose)
    build_proxy(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
