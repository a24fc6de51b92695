"""Builds and runs the C++ unit tests of the placement core (host memcpy hooks + in-process transport), with
AddressSanitizer and UBSan, then exercises the same library through its ctypes binding."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "csrc", "placement")


CORE = ("placement_mapping.cpp", "placement_balancer.cpp", "placement_static.cpp", "placement_manager.cpp")


_CORE_OBJECTS: dict = {}       # sanitizer -> (object files, flags) compiled once per test session


def _core_objects(sanitizer):
    """The library's sources compiled once per sanitizer; every test binary links against the same objects."""
    if sanitizer in _CORE_OBJECTS:
        return _CORE_OBJECTS[sanitizer]
    import tempfile
    out_dir = tempfile.mkdtemp(prefix=f"omni_placement_{sanitizer.replace(',', '_')}_")
    flags = ["-O1", "-g", "-std=c++17", "-Wall", "-pthread", f"-fsanitize={sanitizer}"]
    probe = subprocess.run(["g++", *flags, "-x", "c++", "-", "-o", os.path.join(out_dir, "probe")], input="int main(){return 0;}",
                           capture_output=True, text=True)
    if probe.returncode != 0:
        if sanitizer == "thread":
            _CORE_OBJECTS[sanitizer] = None
            return None
        flags = [f for f in flags if not f.startswith("-fsanitize")]
    objs = []
    procs = []
    for f in CORE:
        o = os.path.join(out_dir, f.replace(".cpp", ".o"))
        procs.append((f, subprocess.Popen(["g++", *flags, "-I", SRC, "-c", os.path.join(SRC, f), "-o", o],
                                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
        objs.append(o)
    for f, pr in procs:
        _, err = pr.communicate()
        assert pr.returncode == 0, f + "\n" + err[-3000:]
    _CORE_OBJECTS[sanitizer] = (objs, flags)
    return _CORE_OBJECTS[sanitizer]


def _build_and_run(tmp_path, name, test_source, sanitizer):
    core = _core_objects(sanitizer)
    if core is None:
        pytest.skip("-fsanitize=thread is not available with this compiler")
    objs, flags = core
    exe = str(tmp_path / name)
    res = subprocess.run(["g++", *flags, "-I", SRC, "-o", exe, os.path.join(SRC, test_source), *objs], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and "ALL PASSED" in run.stdout, run.stdout + run.stderr[-3000:]
    return run


def test_cpp_unit_tests_pass_under_sanitizers(tmp_path):
    _build_and_run(tmp_path, "test_placement", "test_placement.cpp", "address,undefined")


def test_cpp_static_planner_tests_pass_under_sanitizers(tmp_path):
    """Snapshot planner of the static balancer: helpers, instruction semantics, limits, priorities, 300 random cases."""
    _build_and_run(tmp_path, "test_placement_static", "test_placement_static.cpp", "address,undefined")


def test_cpp_unit_cases_per_component(tmp_path):
    """One small case per behaviour of every unit (tensor, mapping, activation, weights + host replica, transports, both
    balancers, optimizer, manager)."""
    import re
    run = _build_and_run(tmp_path, "test_placement_units", "test_placement_units.cpp", "address,undefined")
    m = re.search(r"placement units: (\d+) cases, (\d+) checks, 0 failed", run.stdout)
    assert m and int(m.group(1)) >= 70 and int(m.group(2)) >= 400, run.stdout


def test_cpp_unit_cases_are_race_free_under_thread_sanitizer(tmp_path):
    """The same cases with ThreadSanitizer: the transports, the shared host replica and the manager (ranks as threads,
    background rounds, stop) run several threads."""
    run = _build_and_run(tmp_path, "test_placement_units_tsan", "test_placement_units.cpp", "thread")
    assert "ThreadSanitizer" not in run.stderr, run.stderr[-3000:]


def test_cpp_manager_threads_are_race_free_under_thread_sanitizer(tmp_path):
    """The two-rank round of the manager test runs its ranks as threads over the in-process transport."""
    run = _build_and_run(tmp_path, "test_placement_tsan", "test_placement.cpp", "thread")
    assert "ThreadSanitizer" not in run.stderr, run.stderr[-3000:]
