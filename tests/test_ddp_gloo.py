"""FlexTreeDDP across real processes on CPU: two gloo ranks, the communicator replaced by a stand-in with
the same surface (alloc / all_reduce / world / rank / device) that reduces over gloo.  Checks what a fake
single-rank communicator cannot: every rank launches the same buckets in the same order, parameters start
from rank 0's weights, and the averaged gradients equal those of the whole batch on one process."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP


class GlooComm:
    device = torch.device("cpu")

    def __init__(self):
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.sizes = []

    def alloc(self, shape, dtype=torch.float32):
        return torch.zeros(shape, dtype=dtype)

    def all_reduce(self, t, op="sum", shape=None, algo="auto", **kw):
        self.sizes.append(t.numel())
        dist.all_reduce(t)
        if op == "avg":
            t /= self.world
        return t


def make_model(seed):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(12, 32), nn.GELU(), nn.Linear(32, 32), nn.GELU(), nn.Linear(32, 5))


def worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = GlooComm()
    model = make_model(seed=100 + rank)            # ranks start from different weights on purpose
    ddp = FlexTreeDDP(model, comm, bucket_bytes=2048, broadcast_from=0)
    torch.manual_seed(7)
    x, y = torch.randn(8 * world, 12), torch.randn(8 * world, 5)
    xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
    before = len(comm.sizes)
    with ddp.no_sync():                            # first half of the local batch only accumulates
        nn.functional.mse_loss(ddp(xs[:4]), ys[:4], reduction="sum").backward()
    assert len(comm.sizes) == before
    nn.functional.mse_loss(ddp(xs[4:]), ys[4:], reduction="sum").backward()
    launched = comm.sizes[before:]
    out.put((rank, [p.detach().clone() for p in model.parameters()], [p.grad.detach().clone() for p in model.parameters()],
             launched))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_match_one_process():
    world = 2
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, out)) for r in range(world)]
    [p.start() for p in procs]
    got = sorted((out.get(timeout=120) for _ in range(world)), key=lambda g: g[0])
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    # same weights everywhere, namely rank 0's
    ref = make_model(seed=100)
    for a, b, c in zip(got[0][1], got[1][1], ref.parameters()):
        assert torch.equal(a, b) and torch.allclose(a, c.detach())
    # same buckets in the same order, more than one of them
    assert got[0][3] == got[1][3] and len(got[0][3]) > 1
    # averaged gradients == gradient of (sum of squared errors over the whole batch) / world
    torch.manual_seed(7)
    x, y = torch.randn(8 * world, 12), torch.randn(8 * world, 5)
    nn.functional.mse_loss(ref(x), y, reduction="sum").backward()
    for g0, g1, p in zip(got[0][2], got[1][2], ref.parameters()):
        assert torch.equal(g0, g1)
        assert torch.allclose(g0, p.grad / world, atol=1e-5, rtol=1e-5)
