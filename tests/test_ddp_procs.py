"""FlexTreeDDP on the process world: data-parallel training between ordinary CPU processes with no torch.distributed
and no MPI library at all.  Gradient buckets live in the world's shared heap and are averaged in place."""
import multiprocessing as mp
import uuid

import pytest
import torch
import torch.nn as nn

from test_proc_world import _cross_memory_read_works

pytestmark = pytest.mark.skipif(not _cross_memory_read_works(), reason="process_vm_readv is not available in this sandbox")


def make_model(seed):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(12, 32), nn.GELU(), nn.Linear(32, 32), nn.GELU(), nn.Linear(32, 5))


def worker(rank, world, session, out):
    from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP
    from allreduce_over_mpi_b200.parallel.planner import ProcWorld
    w = ProcWorld(session, rank, world, timeout_s=60)
    w.heap_create(1 << 20)
    model = make_model(seed=100 + rank)                   # different weights per rank on purpose
    ddp = FlexTreeDDP(model, w, bucket_bytes=2048, broadcast_from=0)
    assert all(w.symmetric(b.flat) for b in ddp.buckets)  # the buckets sit at the same heap offsets everywhere
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    torch.manual_seed(7)
    x, y = torch.randn(8 * world, 12), torch.randn(8 * world, 5)
    xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
    for _ in range(3):
        ddp.zero_grad()
        nn.functional.mse_loss(ddp(xs), ys, reduction="sum").backward()
        opt.step()
    out.put((rank, [p.detach().numpy().copy() for p in model.parameters()]))   # by value: the sender exits before the parent reads
    w.barrier()
    ddp.release()
    w.close()


def test_three_processes_train_like_one():
    world = 3
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    session = "ddp-" + uuid.uuid4().hex[:10]
    procs = [ctx.Process(target=worker, args=(r, world, session, out)) for r in range(world)]
    [p.start() for p in procs]
    got = sorted((out.get(timeout=180) for _ in range(world)), key=lambda g: g[0])
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    # one process, whole batch, gradient of the summed loss divided by the world size: the same three steps
    ref = make_model(seed=100)
    opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    torch.manual_seed(7)
    x, y = torch.randn(8 * world, 12), torch.randn(8 * world, 5)
    for _ in range(3):
        ref.zero_grad()
        (nn.functional.mse_loss(ref(x), y, reduction="sum") / world).backward()
        opt.step()
    for a, b, c, r in zip(got[0][1], got[1][1], got[2][1], ref.parameters()):
        assert (a == b).all() and (a == c).all()                # every rank holds the same weights, bit for bit
        assert torch.allclose(torch.from_numpy(a), r.detach(), atol=1e-5, rtol=1e-5)
