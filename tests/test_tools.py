"""Native command-line tools built next to the library (CPU-only invocations)."""
import os
import subprocess

import pytest

from allreduce_over_mpi_b200.build import LIB, ensure_built

BIN = LIB.parent


@pytest.fixture(scope="module", autouse=True)
def built():
    ensure_built()
    for t in ("planner_dump", "cost_model_sweep", "ft_bench"):
        if not (BIN / t).exists():
            pytest.skip(f"{t} not built")


def run(cmd, env=None, cwd=None):
    r = subprocess.run(cmd, capture_output=True, text=True, env={**os.environ, **(env or {})}, cwd=cwd, timeout=120)
    return r.returncode, r.stdout, r.stderr


def test_planner_dump_default_is_the_5_rank_lonely_case():
    rc, out, _ = run([str(BIN / "planner_dump")])
    assert rc == 0
    assert "shape 2*2+1, 4 stages, traffic 216 elements (2*(N-1)*count = 216), race check: clean" in out
    assert "sum b0[0+6] <- 1,4" in out and "get b4[24+3] <- 4" in out
    rc, _, err = run([str(BIN / "planner_dump"), "7", "2,2", "3"])
    assert rc == 1 and "invalid FT_TOPO" in err


def test_cost_model_sweep_prints_reference_choices(tmp_path):
    csv = tmp_path / "numofstru.csv"
    rc, out, _ = run([str(BIN / "cost_model_sweep"), "64", "100", "--csv", str(csv)])
    assert rc == 0
    rows = {int(l.split(",")[0]): l.strip().split(",") for l in csv.read_text().splitlines()[1:]}
    assert rows[8][3] == "1*8" and rows[8][4] == "0.666"
    assert rows[10][3] == "2*5" and rows[50][3] == "2*5*5" and rows[64][3] == "8*8"
    assert rows[12][1] == "9"      # nine candidate shapes for 12 ranks
    assert len(rows) == 64


def test_ft_bench_thread_world_check_and_file(tmp_path):
    exe = str(BIN / "ft_bench")
    rc, out, err = run([exe, "--comm-type", "threads", "--ranks", "6", "--size", "100000", "--repeat", "2", "--check", "--to-file",
                        "--tag", "t"], env={"FT_TOPO": "2,3"}, cwd=tmp_path)
    assert rc == 0, err
    assert "FlexTree enabled" in out and "CHECK (test passed)" in out and "And FlexTree topo is 2*3" in out
    files = [f for f in os.listdir(tmp_path) if f.startswith("t.6.100000.2-3-+0.ar_test.")]
    assert len(files) == 1 and len((tmp_path / files[0]).read_text().split()) == 2
    rc, out, err = run([exe, "--comm-type", "threads", "--ranks", "4", "--size", "35"], env={"FT_TOPO": "2,3"})
    assert rc == 1 and "invalid FT_TOPO 2,3" in err
    rc, out, _ = run([exe, "--version"])
    assert rc == 0 and "FlexTree Standalone Benchmark" in out
    rc, _, err = run([exe, "--bogus"])
    assert rc == 1 and "unknown parameter" in err
    # the two halves as calls of their own, everything a rank does not own wiped in between
    rc, out, err = run([exe, "--comm-type", "threads", "--ranks", "7", "--size", "10007", "--repeat", "2", "--check", "--phases"],
                       env={"FT_TOPO": "2,3", "FT_LONELY": "1"})
    assert rc == 0 and "CHECK (test passed)" in out, err


def test_ft_bench_started_once_per_rank_like_an_mpi_job(tmp_path):
    """--comm-type procs: six copies of the benchmark, one per rank, meet through the process world (no MPI library)."""
    import uuid
    from test_proc_world import _cross_memory_read_works
    if not _cross_memory_read_works():
        pytest.skip("process_vm_readv is not available in this sandbox")
    exe = str(BIN / "ft_bench")
    env = {**os.environ, "FT_WORLD": "6", "FT_SESSION": "tb-" + uuid.uuid4().hex[:8], "FT_TOPO": "2,3"}
    env.pop("FT_LONELY", None)
    ps = [subprocess.Popen([exe, "--comm-type", "procs", "--size", "50000", "--repeat", "2", "--check", "--to-file", "--tag", "p"],
                           env={**env, "FT_RANK": str(r)}, cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
          for r in range(6)]
    outs = [p.communicate(timeout=120) for p in ps]
    assert all(p.returncode == 0 for p in ps), outs
    assert "CHECK (test passed)" in outs[0][0] and "And FlexTree topo is 2*3" in outs[0][0]
    assert all(o[0] == "" for o in outs[1:])                       # only rank 0 talks
    files = [f for f in os.listdir(tmp_path) if f.startswith("p.6.50000.2-3-+0.ar_test.")]
    assert len(files) == 1 and len((tmp_path / files[0]).read_text().split()) == 2


def test_reduce_bench_host_side(tmp_path):
    exe = str(BIN / "reduce_bench")
    rc, out, err = run([exe, "--elements", "50000", "--rounds", "2", "--max-width", "5", "--cpu-only"])
    assert rc == 0, err
    lines = out.strip().splitlines()
    assert all(l.startswith("n=") for l in lines[:5])
    assert len(lines[-1].split()) == 5          # closing line: one average per fan-in
    rc, out, _ = run([exe, "--elements", "1000", "--rounds", "1", "--min-width", "2", "--max-width", "3", "--cpu-only", "--json"])
    import json
    rows = [json.loads(l) for l in out.strip().splitlines()]
    assert [r["n"] for r in rows] == [2, 3] and all(r["cpu_ms"] > 0 for r in rows)
    rc, _, err = run([exe, "--max-width", "33"])
    assert rc == 2 and "max-width" in err


def test_mpi_style_example_builds_and_runs(tmp_path):
    """A program that spells the call MPI_Allreduce compiles against flextree_mpi.h and reduces correctly."""
    import shutil
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    root = BIN.parent.parent
    exe = tmp_path / "mpi_style"
    r = subprocess.run(["g++", "-std=c++17", "-I", str(BIN.parent / "csrc"), str(root / "examples" / "mpi_style.cpp"), "-L", str(BIN),
                        "-lflextree", f"-Wl,-rpath,{BIN}", "-lpthread", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    rc, out, err = run([str(exe), "7"], env={"FT_TOPO": "2,3", "FT_LONELY": "1"})
    assert rc == 0 and "7 ranks, every element = 28 (expected 28): ok" in out, (out, err)
    rc, out, err = run([str(exe), "4"], env={"FT_TOPO": "3,2"})
    assert rc == 1 and "invalid FT_TOPO" in err


def test_cmake_build_of_the_native_library(tmp_path):
    """The CMake route for C/C++ users: configure, build libflextree.so and the tools for sm_100a, run two of them."""
    import shutil
    cmake, gxx = shutil.which("cmake"), shutil.which("g++")
    if not cmake or not gxx or not shutil.which("nvcc"):
        pytest.skip("needs cmake, g++ and nvcc")
    src = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "allreduce_over_mpi_b200", "csrc")
    r = subprocess.run([cmake, "-S", src, "-B", str(tmp_path), f"-DCMAKE_CXX_COMPILER={gxx}", f"-DCMAKE_CUDA_HOST_COMPILER={gxx}"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    r = subprocess.run([cmake, "--build", str(tmp_path), "-j", str(min(8, os.cpu_count() or 2))], capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    flags = (tmp_path / "CMakeFiles" / "flextree.dir" / "flags.make").read_text()
    assert "compute_100a" in flags and "sm_100a" in flags
    rc, out, _ = run([str(tmp_path / "planner_selftest")])
    assert rc == 0 and "selftest ok" in out
    rc, out, err = run([str(tmp_path / "ft_bench"), "--comm-type", "threads", "--ranks", "5", "--size", "1000", "--check"],
                       env={"FT_TOPO": "2,2", "FT_LONELY": "1"})
    assert rc == 0 and "CHECK (test passed)" in out, err


def test_numa_placement_helper_is_best_effort():
    """The helper that moves a benchmark process next to its GPU parses the kernel's CPU lists and does nothing
    (returns None) where the system gives no information, e.g. without a GPU."""
    from allreduce_over_mpi_b200.utils import numa
    assert numa._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert numa._parse_cpulist("") == set()
    import torch
    if not torch.cuda.is_available():
        assert numa.gpu_local_cpus(0) == (set(), None) and numa.bind_to_gpu_node(0) is None


def test_clock_sampler_reads_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The sampler only reads: it starts `nvidia-smi --query-gpu=... -lms`, and summarises median SM clock under load,
    max clock and the throttle reasons seen.  Here the program on PATH is a script that prints three samples."""
    import os
    import stat
    import time
    from allreduce_over_mpi_b200.utils.clocks import ClockSampler
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\n"
                    "echo '0, 1965, 1965, 120.5, 0x0, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo '0, 1710, 1965, 940.0, 0x4, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1650, 1965, 950.0, 0x4, Not Active, Not Active, Not Active, Active'\n"
                    "echo 'garbage line'\n"
                    "sleep 30\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    s = ClockSampler(gpu_index=0).start()
    time.sleep(0.5)
    name = s._file.name
    got = s.stop()
    assert got["samples"] == 3 and got["sm_max_mhz"] == 1965.0 and got["reasons"] == ["sw_power_cap"]
    assert got["sm_mhz"] == 1680.0 and got["power_w_max"] == 950.0      # median of the two samples under load
    assert not os.path.exists(name)                                      # the sample file is removed
    monkeypatch.setenv("PATH", str(tmp_path / "nowhere"))
    assert ClockSampler().start().stop()["samples"] == 0                 # no nvidia-smi: an empty record, no error
