"""Process-per-rank world on CPU: ranks are ordinary processes of this host (no MPI library, no torch.distributed);
blocks are pulled out of the peers' buffers with process_vm_readv, small messages go through the shared segment."""
import multiprocessing as mp
import os
import subprocess
import uuid

import pytest
import torch

from allreduce_over_mpi_b200.build import LIB


def _cross_memory_read_works() -> bool:
    """process_vm_readv is filtered out in some sandboxes (it needs no privilege for one's own processes, but a
    system-call filter can remove it altogether): probe it on this process's own memory."""
    import ctypes as C

    class IOVec(C.Structure):
        _fields_ = [("base", C.c_void_p), ("len", C.c_size_t)]
    try:
        libc = C.CDLL(None, use_errno=True)
        src, dst = C.create_string_buffer(b"probe-ok", 8), C.create_string_buffer(8)
        lv, rv = IOVec(C.addressof(dst), 8), IOVec(C.addressof(src), 8)
        libc.process_vm_readv.restype = C.c_ssize_t
        got = libc.process_vm_readv(os.getpid(), C.byref(lv), 1, C.byref(rv), 1, 0)
        return got == 8 and dst.raw == b"probe-ok"
    except Exception:  # noqa: BLE001
        return False


pytestmark = pytest.mark.skipif(not _cross_memory_read_works(), reason="process_vm_readv is not available in this sandbox")


def _rank(rank, world, session, topo, lonely, q):
    os.environ.pop("FT_TOPO", None); os.environ.pop("FT_LONELY", None)
    if topo:
        os.environ["FT_TOPO"] = topo
    if lonely:
        os.environ["FT_LONELY"] = lonely
    from allreduce_over_mpi_b200.parallel.planner import ProcWorld
    w = ProcWorld(session, rank, world, timeout_s=60)
    ok = True
    for count, dtype in ((35, torch.float32), (3000, torch.float64), (300_007, torch.float32), (70_001, torch.int32)):
        for rep in range(2):                       # back to back: flags keep growing, buffers are reused
            g = torch.Generator().manual_seed(1000 * rep + count)
            every = [(torch.rand(count, generator=g, dtype=torch.float64) * 200 - 100).to(dtype) for _ in range(world)]
            mine = every[rank].clone()
            w.all_reduce(mine)
            want = torch.stack([e.double() for e in every]).sum(0)
            ok = ok and torch.allclose(mine.double(), want, rtol=1e-5, atol=1e-3)
            src, dst = every[rank].clone(), torch.zeros(count, dtype=dtype)
            w.all_reduce(src, out=dst)             # out of place leaves the source alone
            ok = ok and torch.equal(src, every[rank]) and torch.equal(dst, mine)
    # tensors in the world's symmetric heap: reduced in place through the peers' shared mappings
    w.heap_create(4 << 20)
    a, b = w.alloc(200_003, torch.float32), w.alloc((50, 7), torch.float64)
    ok = ok and w.symmetric(a) and w.symmetric(b)
    for rep in range(2):
        g = torch.Generator().manual_seed(77 + rep)
        every = [torch.rand(200_003, generator=g) * 2 - 1 for _ in range(world)]
        a.copy_(every[rank])
        w.all_reduce(a)
        ok = ok and torch.allclose(a.double(), torch.stack([e.double() for e in every]).sum(0), atol=1e-4)
        b.fill_(float(rank + 1))
        w.all_reduce(b)
        ok = ok and bool((b == world * (world + 1) / 2).all())
    # the two halves as calls of their own, on private memory and on a heap tensor; what a rank does not own is
    # overwritten in between
    for t in (torch.empty(90_001, dtype=torch.float64), w.alloc(90_001, torch.float64)):
        t.fill_(float(rank + 1))
        mine = w.reduce_scatter(t)
        ok = ok and len(mine) == 1 and bool((mine[0] == world * (world + 1) / 2).all())
        keep = mine[0].clone()
        t.fill_(float("nan"))
        mine[0].copy_(keep)
        w.all_gather(t)
        ok = ok and bool((t == world * (world + 1) / 2).all())
    times = w.profile_phases(torch.ones(50_000), iters=2)
    ok = ok and times["reduce_scatter_ms"] > 0 and times["all_gather_ms"] > 0
    w.free(b)
    c = w.alloc(300, torch.float64)
    ok = ok and c.data_ptr() == b.data_ptr() and w.symmetric(c)      # first fit: the freed block is handed out again
    w.barrier()
    w.close()
    q.put((rank, ok))


@pytest.mark.parametrize("world,topo,lonely", [(2, None, None), (6, "2,3", None), (7, "2,3", "1"), (5, "1", None), (8, "2,2,2", None)])
def test_processes_all_reduce(world, topo, lonely):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    session = "t-" + uuid.uuid4().hex[:10]
    ps = [ctx.Process(target=_rank, args=(r, world, session, topo, lonely, q)) for r in range(world)]
    [p.start() for p in ps]
    got = dict(q.get(timeout=180) for _ in range(world))
    [p.join(timeout=60) for p in ps]
    assert got == {r: True for r in range(world)}
    assert all(p.exitcode == 0 for p in ps)
    assert not os.path.exists(f"/dev/shm/ftpw-{session}")       # the last rank out removed the segment


def test_a_rank_that_never_joins_is_a_timeout_not_a_hang():
    from allreduce_over_mpi_b200 import FlexTreeError
    from allreduce_over_mpi_b200.parallel.planner import ProcWorld
    session = "t-" + uuid.uuid4().hex[:10]
    with pytest.raises(FlexTreeError, match="not every rank joined"):
        ProcWorld(session, 0, 2, timeout_s=0.5)
    try:
        os.unlink(f"/dev/shm/ftpw-{session}")
    except OSError:
        pass


def test_mpi_spelled_program_as_processes(tmp_path):
    """examples/mpi_style_procs.cpp: MPI names, one process per rank, 2*3+1 lonely layout, no MPI library."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = tmp_path / "mpi_style_procs"
    r = subprocess.run(["g++", "-std=c++17", "-I", os.path.join(root, "allreduce_over_mpi_b200", "csrc"),
                        os.path.join(root, "examples", "mpi_style_procs.cpp"), "-L", str(LIB.parent), "-lflextree",
                        f"-Wl,-rpath,{LIB.parent}", "-lpthread", "-o", str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    session = "t-" + uuid.uuid4().hex[:10]
    env = dict(os.environ, FT_WORLD="7", FT_SESSION=session, FT_TOPO="2,3", FT_LONELY="1")
    ps = [subprocess.Popen([str(exe)], env=dict(env, FT_RANK=str(k)), stdout=subprocess.PIPE, text=True) for k in range(7)]
    outs = [p.communicate(timeout=120)[0] for p in ps]
    assert all(p.returncode == 0 for p in ps), outs
    assert sorted(outs) == [f"rank {k} of 7: every element = 28 (expected 28): ok\n" for k in range(7)]


def test_launcher_starts_one_copy_per_rank_and_reports_the_worst_exit_code():
    """python -m allreduce_over_mpi_b200.parallel.launch: the one-host stand-in for mpirun."""
    import sys
    import time
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(LIB.parent / "ft_bench")
    r = subprocess.run([sys.executable, "-m", "allreduce_over_mpi_b200.parallel.launch", "-np", "5", "--topo", "2,2", "--lonely", "1", "--",
                        exe, "--comm-type", "procs", "--size", "20000", "--repeat", "2", "--check"],
                       capture_output=True, text=True, timeout=120, cwd=root)
    assert r.returncode == 0 and "CHECK (test passed)" in r.stdout and "topo is 2*2+1" in r.stdout, (r.stdout, r.stderr)
    t0 = time.time()   # one rank fails at once: the job ends with its code and the others are stopped, not waited for
    r = subprocess.run([sys.executable, "-m", "allreduce_over_mpi_b200.parallel.launch", "-np", "3", "--", "sh", "-c",
                        "test $FT_RANK != 1 || exit 7; sleep 30"], capture_output=True, text=True, timeout=60, cwd=root)
    assert r.returncode == 7 and time.time() - t0 < 20
