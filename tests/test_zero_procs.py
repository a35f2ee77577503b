"""Optimizer state split over the ranks (reduce-scatter of the gradients, all-gather of the parameters) on the process
world: three CPU processes train like one process with the whole batch, and each holds about a third of Adam's state."""
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


CLIP = 0.5     # below the gradient norm of the first steps, so that clipping really scales


def make_opt(params):
    return torch.optim.AdamW(params, lr=0.01, weight_decay=0.0)


def worker(rank, world, session, shape, out):
    from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP
    from allreduce_over_mpi_b200.parallel.planner import ProcWorld
    from allreduce_over_mpi_b200.parallel.zero import ShardedOptimizer
    w = ProcWorld(session, rank, world, timeout_s=60)
    w.heap_create(1 << 20)
    model = make_model(seed=100 + rank)                   # different weights per rank on purpose
    ddp = FlexTreeDDP(model, w, bucket_bytes=2048, broadcast_from=0, sharded=True, shape=shape)
    opt = ShardedOptimizer(ddp, make_opt)
    assert all(w.symmetric(t) for t in opt.param_flats)
    torch.manual_seed(7)
    x, y = torch.randn(8 * world, 12), torch.randn(8 * world, 5)
    xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
    norms = []
    for _ in range(4):
        opt.zero_grad()
        nn.functional.mse_loss(ddp(xs), ys, reduction="sum").backward()
        norms.append(float(opt.clip_grad_norm_(CLIP)))
        opt.step()
    sd = opt.state_dict()
    opt.load_state_dict(sd)                               # round trip of this rank's part
    owned = sum(hi - lo for rng in opt.ranges for lo, hi in rng)
    out.put((rank, [p.detach().numpy().copy() for p in model.parameters()], owned, opt.state_elements(), norms))
    w.barrier()
    opt.release()
    ddp.release()
    w.close()


@pytest.mark.parametrize("shape", [None, "ring3"])     # flat tree: rank r owns block r; ring: block r + 1
def test_three_processes_with_split_adam_state_train_like_one(shape):
    world = 3
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    session = "zero-" + uuid.uuid4().hex[:10]
    procs = [ctx.Process(target=worker, args=(r, world, session, shape, out)) for r in range(world)]
    [p.start() for p in procs]
    got = sorted((out.get(timeout=180) for _ in range(world)), key=lambda g: g[0])
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    ref = make_model(seed=100)
    opt = make_opt(ref.parameters())
    torch.manual_seed(7)
    x, y = torch.randn(8 * world, 12), torch.randn(8 * world, 5)
    ref_norms = []
    for _ in range(4):
        ref.zero_grad()
        (nn.functional.mse_loss(ref(x), y, reduction="sum") / world).backward()
        ref_norms.append(float(torch.nn.utils.clip_grad_norm_(ref.parameters(), CLIP)))
        opt.step()
    assert ref_norms[0] > CLIP                                   # the clip was active
    for g in got:
        assert all(abs(a - b) <= 1e-4 * max(1.0, b) for a, b in zip(g[4], ref_norms)), (g[4], ref_norms)
    for a, b, c, r in zip(got[0][1], got[1][1], got[2][1], ref.parameters()):
        assert (a == b).all() and (a == c).all()                # every rank holds the same weights, bit for bit
        assert torch.allclose(torch.from_numpy(a), r.detach(), atol=2e-5, rtol=1e-4)
    total = sum(p.numel() for p in ref.parameters())
    owned = [g[2] for g in got]
    assert sum(owned) >= total and max(owned) < 0.6 * total      # the buckets' padding is owned too; nobody holds most of it
    for g in got:
        assert 2 * g[2] <= g[3] <= 2 * g[2] + 64                 # two moments per owned element, plus Adam's step counters
