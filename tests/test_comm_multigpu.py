"""Multi-process, multi-GPU runs of the communicator (one process per GPU under
torch.distributed.run).  Skipped on boxes with fewer than two GPUs."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def run_worker(nproc, mode, env_extra=None, port=29541, timeout=900):
    env = dict(os.environ)
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "mp_comm_worker.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, f"rc={r.returncode}\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return json.loads(lines[-1][7:])


def ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("nproc", [2, 3, 4, 5, 6, 7, 8])
def test_all_shapes_all_algorithms(nproc):
    if ngpu() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    res = run_worker(nproc, "correctness", port=29540 + nproc)
    assert res["ok"], res
    assert res["cases"] > 20


def test_ipc_memory_kind():
    if ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_worker(2, "correctness", {"FT_MEM": "ipc"}, port=29561)
    assert res["ok"] and res["mem_kind"] == 0 and not res["nvls"], res


def test_absent_rank_times_out_instead_of_hanging():
    """A rank that skips a call: the others' device-side waits run out and report a status; nothing
    hangs or faults.  NVLS stays off for this one (plain peer loads only)."""
    n = min(ngpu(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    res = run_worker(n, "timeout", {"FT_NVLS": "0", "NCCL_NVLS_ENABLE": "0"}, port=29571)
    assert res["ok"], res
