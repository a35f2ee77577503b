"""The host-only core (planner, cost models, CPU executors) under AddressSanitizer +
UndefinedBehaviorSanitizer and, for the thread-per-rank executor, ThreadSanitizer."""
import shutil
import subprocess
from pathlib import Path

import pytest

SRC = Path(__file__).resolve().parents[1] / "allreduce_over_mpi_b200" / "csrc" / "tools" / "planner_selftest.cpp"


def build_and_run(tmp_path, flags, args):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = tmp_path / "selftest"
    r = subprocess.run(["g++", "-std=c++17", "-O1", "-g", *flags, str(SRC), "-o", str(exe), "-lpthread"], capture_output=True, text=True)
    if r.returncode != 0 and "sanitize" in r.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert r.returncode == 0, r.stderr[-2000:]
    r = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "selftest ok" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
    assert "ERROR: AddressSanitizer" not in r.stderr and "WARNING: ThreadSanitizer" not in r.stderr and "runtime error" not in r.stderr


def test_asan_ubsan(tmp_path):
    build_and_run(tmp_path, ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], [])


def test_tsan_thread_world(tmp_path):
    build_and_run(tmp_path, ["-fsanitize=thread"], ["threads"])


def test_range_predicate_of_the_bounds_checked_build():
    """The test the FT_BOUNDS build of the kernels applies to every run of heap bytes before touching it, evaluated
    on the host: its failing branch is exercised here and never on a GPU."""
    from allreduce_over_mpi_b200._lib import lib
    ok = lib().ft_bounds_check_host
    heap = 1 << 20
    assert ok(heap, 0, 8, 0, heap) == 1 and ok(heap, 7, 8, heap - 16, 16) == 1 and ok(heap, 3, 8, heap, 0) == 1
    assert ok(heap, 0, 8, heap - 16, 32) == 0          # runs past the end
    assert ok(heap, 0, 8, heap + 1, 0) == 0            # starts past the end
    assert ok(heap, 8, 8, 0, 16) == 0 and ok(heap, -1, 8, 0, 16) == 0      # no such rank
    assert ok(heap, 0, 8, (1 << 64) - 8, 16) == 0      # offset + length would wrap around
    assert ok(0, 0, 1, 0, 1) == 0
