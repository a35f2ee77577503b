"""The benchmark's reference arm at N > 1 runs on CPU (the reference has no GPU data path):
unmodified benchmark.cpp + mpi_mod.hpp over the shared-memory MPI shim, one process per rank."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_BIN = os.path.join(ROOT, "baseline", "_ref", "ref_mpi_bench")


@pytest.mark.skipif(not os.path.exists(REF_BIN), reason="reference not built (python baseline/install_reference.py)")
@pytest.mark.parametrize("world,topo,lonely", [(2, None, None), (6, "2,3", None), (7, "2,3", "1")])
def test_reference_arm_multi_rank(world, topo, lonely):
    env = dict(os.environ)
    env.pop("FT_TOPO", None); env.pop("FT_LONELY", None)
    if topo:
        env["FT_TOPO"] = topo
    if lonely:
        env["FT_LONELY"] = lonely
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29800 + world), os.path.join(ROOT, "bench.py"), "--gpus", str(world), "--steps", "3", "--warmup", "3",
           "--bytes", str(4 << 20), "--impl", "reference"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0 and len(lines) == 1, (r.stdout[-1500:], r.stderr[-1500:])
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and "unavailable" not in out, out
    assert out["n_gpus"] == world and out["value"] > 0 and out["details"]["FT_TOPO"] == (topo or str(world))
    assert not os.path.exists(f"/dev/shm/ftshim-{29800 + world}")      # the shim removed its segment


def test_reference_arm_single_gpu_reports_unavailable_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("has a GPU")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True, text=True, timeout=120)
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert r.returncode == 0 and out["impl"] == "reference" and "unavailable" in out


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "baseline", "_ref", "ref_config1")),
                    reason="reference not built (python baseline/install_reference.py)")
def test_seeded_fp64_checked_comparison_on_6_and_7_ranks():
    """World 6 (2*3) and 7 (2*3 + 1 lonely), uniform[-1,1) data from seed = rank, fp64 oracle:
    the unmodified reference, the thread world and the process world (ranks launched as processes, like the
    reference's) all pass and report a time."""
    from test_proc_world import _cross_memory_read_works
    procs = _cross_memory_read_works()
    r = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "config1.py"), "--count", "20000", "--repeat", "3",
                        "--warmup", "1", "--omp", "1"] + ([] if procs else ["--no-procs"]), capture_output=True, text=True, timeout=300, cwd=ROOT)
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    arms = ["reference", "flextree-threads"] + (["flextree-procs", "flextree-procs-heap"] if procs else [])
    assert r.returncode == 0 and len(rows) == 2 * len(arms), (r.stdout[-1500:], r.stderr[-1500:])
    assert [(d["impl"], d["world"]) for d in rows] == [(a, 6) for a in arms] + [(a, 7) for a in arms]
    assert all(d["check"] == "passed" and d["ms_min"] > 0 for d in rows)
    assert rows[-1]["FT_LONELY"] == "1" and rows[1]["FT_TOPO"] == "2,3"
