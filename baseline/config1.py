"""CPU all-reduce on the reference's own ground: world 6 as a 2*3 tree and world 7 as 2*3 plus one
lonely rank, 1 048 576 floats per rank drawn uniform[-1,1) from seed = rank, result checked against
an fp64 sum.  Both arms run config1_driver.cpp (built by install_reference.py):

  reference   unmodified mpi_mod.hpp (MPI_Allreduce_FT) over the shared-memory MPI shim, one
              process per rank.  Its reduction loops ask for 14 OpenMP threads in the source
              (PARALLEL_THREAD, mpi_mod.hpp:820), which oversubscribes a small machine, so it is
              run both as it is and with OMP_THREAD_LIMIT=1 and the faster run is reported
  flextree    this repository's MPI-compatible entry over the thread world (one thread per rank) and over the
              process world (one process per rank, launched like the reference arm; no MPI library underneath),
              the latter with the tensor in private memory and in the world's symmetric shared heap

    python baseline/config1.py [--count 1048576] [--repeat 20] [--warmup 3]

Prints one JSON line per (arm, world).  Neither arm touches a GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import uuid

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
CASES = ((6, "2,3", None), (7, "2,3", "1"))


def _env(topo, lonely, **extra):
    env = {k: v for k, v in os.environ.items() if k not in ("FT_TOPO", "FT_LONELY")}
    env["FT_TOPO"] = topo
    if lonely:
        env["FT_LONELY"] = lonely
    env.update(extra)
    return env


def run_flextree(world, topo, lonely, count, repeat, warmup):
    r = subprocess.run([os.path.join(REF, "ft_config1"), str(world), str(count), str(repeat), str(warmup)],
                       capture_output=True, text=True, env=_env(topo, lonely), timeout=600)
    if r.returncode != 0:
        return {"impl": "flextree-threads", "world": world, "error": r.stderr[-300:]}
    return json.loads(r.stdout.strip().splitlines()[-1])


def run_flextree_procs(world, topo, lonely, count, repeat, warmup, heap=False):
    session = "c1p-" + uuid.uuid4().hex[:10]
    procs = []
    for rank in range(world):
        env = _env(topo, lonely, FT_RANK=str(rank), FT_WORLD=str(world), FT_SESSION=session, CONFIG1_HEAP="1" if heap else "0")
        procs.append(subprocess.Popen([os.path.join(REF, "ft_config1_procs"), str(world), str(count), str(repeat), str(warmup)],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, env=env))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=600)[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        try:
            os.unlink(f"/dev/shm/ftpw-{session}")
        except OSError:
            pass
    if any(p.returncode for p in procs):
        return {"impl": "flextree-procs-heap" if heap else "flextree-procs", "world": world, "error": f"exit codes {[p.returncode for p in procs]}"}
    return json.loads(outs[0].strip().splitlines()[-1])


def run_reference(world, topo, lonely, count, repeat, warmup, thread_limit):
    session = "c1-" + uuid.uuid4().hex[:10]
    procs = []
    for rank in range(world):
        env = _env(topo, lonely, FTSHIM_RANK=str(rank), FTSHIM_SIZE=str(world), FTSHIM_SESSION=session)
        env.pop("OMP_THREAD_LIMIT", None)
        if thread_limit:   # 0 = the reference as it is (14 threads per reduction loop)
            env["OMP_THREAD_LIMIT"] = str(thread_limit)
        procs.append(subprocess.Popen([os.path.join(REF, "ref_config1"), str(world), str(count), str(repeat), str(warmup)],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, env=env))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=600)[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        try:
            os.unlink(f"/dev/shm/ftshim-{session}")
        except OSError:
            pass
    if any(p.returncode for p in procs):
        return {"impl": "reference", "world": world, "error": f"exit codes {[p.returncode for p in procs]}"}
    d = json.loads(outs[0].strip().splitlines()[-1])
    d["omp_thread_limit"] = thread_limit or "unset (14 threads per loop)"
    return d


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--count", type=int, default=1 << 20)
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--omp", type=int, nargs="+", default=[0, 1], help="OMP_THREAD_LIMIT values tried for the reference (0 = unset)")
    ap.add_argument("--no-procs", action="store_true", help="leave the process-world arms out (sandboxes without process_vm_readv)")
    a = ap.parse_args(argv)
    for exe in ("ref_config1", "ft_config1"):
        if not os.path.exists(os.path.join(REF, exe)):
            print(json.dumps({"unavailable": f"baseline/_ref/{exe} is not built (run python baseline/install_reference.py)"}))
            return 0
    bad = 0
    for world, topo, lonely in CASES:
        refs = [run_reference(world, topo, lonely, a.count, a.repeat, a.warmup, t) for t in a.omp]
        good = [r for r in refs if "error" not in r]
        ref = min(good, key=lambda r: r["ms_min"]) if good else refs[0]
        ours = run_flextree(world, topo, lonely, a.count, a.repeat, a.warmup)
        rows = [ref, ours]
        if os.path.exists(os.path.join(REF, "ft_config1_procs")) and not a.no_procs:
            rows.append(run_flextree_procs(world, topo, lonely, a.count, a.repeat, a.warmup))
            rows.append(run_flextree_procs(world, topo, lonely, a.count, a.repeat, a.warmup, heap=True))
        for d in rows[1:]:
            if "error" not in ref and "error" not in d:
                d["speedup_vs_reference_at_min"] = round(ref["ms_min"] / d["ms_min"], 2)
        for d in rows:
            bad += "error" in d or d.get("check") != "passed"
            print(json.dumps(d))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
