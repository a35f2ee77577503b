"""Start a program once per rank on this host, the way ``mpirun -np N`` starts an MPI job:

    python -m allreduce_over_mpi_b200.parallel.launch -np 6 [--topo 2,3] [--lonely 1] -- <program> [args ...]

Every copy gets FT_RANK, FT_WORLD and a fresh FT_SESSION (plus RANK / WORLD_SIZE / LOCAL_RANK for programs that read
those), which is all ``ft_mpi_proc_init_env`` / ``planner.ProcWorld()`` need to find each other.  Output is passed
through; the exit code is the largest of the ranks'; when one rank fails the others are stopped.  The reference
is started with ``mpirun --hostfile mpi_config_file`` across 16 hosts (allreduce_over_mpi/Makefile:8-24,
mpi_config_file:1-16); this launcher covers one host, the scope of the process world.
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time
import uuid


def launch(cmd: list[str], nprocs: int, topo: str | None = None, lonely: str | None = None, env: dict | None = None,
           timeout: float | None = None) -> int:
    base = dict(os.environ if env is None else env)
    base.update(FT_WORLD=str(nprocs), WORLD_SIZE=str(nprocs), FT_SESSION="job-" + uuid.uuid4().hex[:12])
    if topo is not None:
        base["FT_TOPO"] = topo
    if lonely is not None:
        base["FT_LONELY"] = lonely
    # every rank leads a process group of its own, so that stopping a rank also stops what it started
    procs = [subprocess.Popen(cmd, env={**base, "FT_RANK": str(r), "RANK": str(r), "LOCAL_RANK": str(r)}, start_new_session=True)
             for r in range(nprocs)]

    def stop(p, sig):
        try:
            os.killpg(p.pid, sig)      # the group led by the process started above, nothing else
        except (ProcessLookupError, PermissionError):
            pass
    t0 = time.monotonic()
    worst = 0
    try:
        while True:
            codes = [p.poll() for p in procs]          # poll every rank, every time
            if all(c is not None for c in codes):
                break
            failed = [c for c in codes if c not in (None, 0)]
            if failed or (timeout is not None and time.monotonic() - t0 > timeout):
                worst = max([abs(c) for c in failed] + [124 if not failed else 0])
                break
            time.sleep(0.01)
    finally:
        stopped_early = any(p.poll() is None for p in procs)
        for p in procs:
            if p.poll() is None or stopped_early:
                stop(p, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                stop(p, signal.SIGKILL)
                p.wait()
    try:
        os.unlink("/dev/shm/ftpw-" + base["FT_SESSION"])   # a job that was stopped half-way leaves its control segment
    except OSError:
        pass
    return max([worst] + [abs(p.returncode or 0) for p in procs if worst == 0])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-np", "--nprocs", type=int, required=True)
    ap.add_argument("--topo", default=None, help="FT_TOPO for the job (bottom-up widths, e.g. 2,3)")
    ap.add_argument("--lonely", default=None, help="FT_LONELY for the job")
    ap.add_argument("--timeout", type=float, default=None, help="stop the job after this many seconds")
    ap.add_argument("cmd", nargs=argparse.REMAINDER, help="-- program [args ...]")
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd[:1] == ["--"] else a.cmd
    if not cmd or a.nprocs < 1:
        ap.error("give -np N and a program after --")
    return launch(cmd, a.nprocs, a.topo, a.lonely, timeout=a.timeout)


if __name__ == "__main__":
    sys.exit(main())
