"""Further single-GPU tests of the communicator (ranks emulated stage by stage on one stream, no kernel
waits on another): the two halves of the plan as collectives of their own, guard blocks behind heap
tensors, odd-offset slices of heap tensors, and the heap allocator's free / reuse."""
import pytest
import torch

from allreduce_over_mpi_b200.parallel import planner as P
from allreduce_over_mpi_b200.parallel.comm import LocalWorld
from allreduce_over_mpi_b200.parallel.planner import Shape

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def inputs(world, count, dtype, seed=0):
    out = []
    for r in range(world):
        g = torch.Generator().manual_seed(seed * 100 + r)
        x = torch.rand(count, generator=g, dtype=torch.float64) * 2 - 1
        out.append(x.to(dtype) if dtype.is_floating_point else (x * 50).to(dtype))
    return out


def tol(dtype):
    return {torch.float32: 1e-5, torch.float64: 1e-12, torch.bfloat16: 0.15, torch.float16: 0.02}.get(dtype, 0)


@pytest.mark.parametrize("text", ["2", "4", "2*2+1", "2*4", "2*2*2", "ring5", "3*2+1", "8"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_scatter_and_all_gather_alone(text, dtype):
    """The two halves of the staged plan as collectives of their own: after reduce_scatter a rank's
    own block is complete (everything it does not own is then overwritten with NaN), and all_gather
    alone rebuilds the full result from the owned blocks."""
    shape = Shape.parse(text)
    n = shape.world
    w = LocalWorld(n, heap_bytes=8 << 20, staging_bytes=1 << 16)
    for count in (5, 4099, 300_001):
        host = inputs(n, count, dtype, seed=11)
        want = torch.stack(host).double().sum(0) / n
        dev = []
        for r, c in enumerate(w.ranks):
            t = c.alloc(count, dtype)
            t.copy_(host[r])
            dev.append(t)
        owned = w.reduce_scatter(dev, op="avg", shape=shape)
        torch.cuda.synchronize()
        covered = torch.zeros(count, dtype=torch.bool)
        for r, c in enumerate(w.ranks):
            blocks = P.owned_blocks(n, shape, r)
            assert len(blocks) == 1 and len(owned[r]) == 1
            lo, hi = c.block_range(dev[r], blocks[0])
            assert owned[r][0].numel() == hi - lo and (hi == lo or owned[r][0].data_ptr() == dev[r][lo:hi].data_ptr())
            assert torch.allclose(dev[r][lo:hi].double().cpu(), want[lo:hi], atol=tol(dtype)), (text, count, r)
            covered[lo:hi] = True
            keep = dev[r][lo:hi].clone()
            dev[r].fill_(float("nan"))
            dev[r][lo:hi] = keep
        assert bool(covered.all())
        w.all_gather(dev, shape=shape)
        torch.cuda.synchronize()
        for r in range(n):
            assert torch.allclose(dev[r].double().cpu(), want, atol=tol(dtype)), (text, count, r)
        assert all(torch.equal(d, dev[0]) for d in dev)
        for c in w.ranks:
            c.free_all()
    w.close()


def test_phases_refuse_tensors_outside_the_heap():
    w = LocalWorld(2, heap_bytes=1 << 20, staging_bytes=1 << 16)
    outside = [torch.zeros(64, device=DEV) for _ in range(2)]
    with pytest.raises(ValueError):
        w.reduce_scatter(outside)
    w.close()


def test_guard_blocks_behind_heap_tensors_stay_intact():
    """Opt-in canaries: a 256-byte guard of a known pattern behind every heap tensor.  No collective
    kernel may touch them, whatever the length (odd sizes put the tensor's end in the middle of a
    16-byte vector and of a lane's slice); a write into a guard is reported."""
    n = 5
    w = LocalWorld(n, heap_bytes=8 << 20, staging_bytes=1 << 20)
    for c in w.ranks:
        c.enable_canaries()
    for count in (1, 333, 4099, 250_001):
        for dtype in (torch.float32, torch.bfloat16):
            dev = []
            for r, c in enumerate(w.ranks):
                t = c.alloc(count, dtype)
                t.fill_(1.0)
                dev.append(t)
            for shape in ("5", "2*2+1", "ring5"):
                w.all_reduce(dev, op="avg", shape=shape)
                w.reduce_scatter(dev, shape=shape, op="avg")
                w.all_gather(dev, shape=shape)
            w.all_reduce(dev, op="avg", algo="push")
            torch.cuda.synchronize()
            for r, c in enumerate(w.ranks):
                assert c.check_canaries() >= 1
    # a write that does run past a tensor is caught (done here with an ordinary torch copy into the guard)
    guard = w.ranks[2]._canaries[-1][0]
    guard[:4] = 0
    with pytest.raises(Exception, match="overwritten"):
        w.ranks[2].check_canaries()
    w.close()


def test_unaligned_slice_of_a_heap_tensor_goes_through_the_slots():
    """A view that starts at an odd element of a heap tensor is not on a 16-byte boundary: it must not be
    addressed in place with vector loads.  It is reduced like any user tensor, and the elements around it
    stay as they were."""
    w = LocalWorld(4, heap_bytes=1 << 20, staging_bytes=1 << 20)
    host = inputs(4, 3001, torch.float32, seed=21)
    want = torch.stack(host).double().sum(0)
    base, views = [], []
    for r, c in enumerate(w.ranks):
        b = c.alloc(3010, torch.float32)
        b.fill_(-7.0)
        v = b[3:3 + 3001]
        assert c.in_heap(b) and not c.in_heap(v)
        v.copy_(host[r])
        base.append(b); views.append(v)
    for shape in ("4", "2*2"):
        w.all_reduce(views, shape=shape)
        torch.cuda.synchronize()
        for r in range(4):
            assert torch.allclose(views[r].double().cpu(), want, atol=1e-5), (shape, r)
            assert bool((base[r][:3] == -7).all()) and bool((base[r][3 + 3001:] == -7).all())
        for v, h in zip(views, host):
            v.copy_(h)
    with pytest.raises(Exception, match="symmetric heap"):
        w.all_reduce(views, algo="push")
    w.close()


def test_heap_free_and_reuse():
    """alloc / free: a freed block is handed out again (first fit at the lowest offset, the same on every
    rank), freed neighbours merge, and a collective on the reused block works."""
    w = LocalWorld(3, heap_bytes=1 << 20, staging_bytes=1 << 16)
    ptrs = []
    for c in w.ranks:
        a, b, d = c.alloc(1000), c.alloc(5000), c.alloc(1000)
        hole = b.data_ptr() - a.data_ptr()
        assert hole == 4096 and d.data_ptr() - b.data_ptr() == 20224      # 4000 B -> 4096, 20000 B -> 20224
        before = c.heap_free_bytes
        c.free(b)
        e = c.alloc(4000)
        assert e.data_ptr() == b.data_ptr() and c.heap_free_bytes == before
        with pytest.raises(Exception, match="ft_comm_free"):
            c.free(e[1:])                      # not the start of a block
        c.free(a); c.free(e)                   # neighbours merge: one block of 4096 + 20224 bytes at the start
        f = c.alloc(6000)
        assert f.data_ptr() == a.data_ptr()
        ptrs.append(f)
    host = inputs(3, 6000, torch.float32, seed=31)
    for t, h in zip(ptrs, host):
        t.copy_(h)
    w.all_reduce(ptrs, shape="3")
    torch.cuda.synchronize()
    want = torch.stack(host).double().sum(0)
    assert all(torch.allclose(t.double().cpu(), want, atol=1e-5) for t in ptrs)
    w.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int32])
def test_world_of_one_scales_every_float_type_like_larger_worlds(dtype):
    """op="avg"-style scaling at world 1: every floating type is scaled (an odd length and an odd offset take the
    element-wise tail), integers never are - the same numbers a larger world's kernels would give."""
    w = LocalWorld(1, heap_bytes=1 << 20, staging_bytes=1 << 16)
    c = w.ranks[0]
    for count, off in ((1, 0), (4099, 0), (70_003, 1)):
        base = torch.arange(count + off, device=DEV).remainder(97).to(dtype)
        x = base[off:].clone() if off == 0 else base[off:]
        want = x.double() * (0.25 if dtype.is_floating_point else 1.0)
        c.all_reduce(x, scale=0.25)
        torch.cuda.synchronize()
        assert (x.double() - want).abs().max().item() <= tol(dtype) * 10, (dtype, count)
    h = c.alloc(1000, dtype)
    h.fill_(8)
    c.reduce_scatter(h, scale=0.5)
    c.all_gather(h)
    torch.cuda.synchronize()
    assert bool((h == (4 if dtype.is_floating_point else 8)).all())
    w.close()


def test_split_optimizer_state_on_a_world_of_one():
    """The optimizer with split state on a single rank owns everything: same parameters as a plain AdamW, the module's
    parameters living in the communicator's heap meanwhile and in ordinary memory again after release()."""
    import torch.nn as nn
    from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP
    from allreduce_over_mpi_b200.parallel.zero import ShardedOptimizer

    def make():
        torch.manual_seed(3)
        return nn.Sequential(nn.Linear(24, 48), nn.GELU(), nn.Linear(48, 7)).to(DEV)

    w = LocalWorld(1, heap_bytes=4 << 20, staging_bytes=1 << 16)
    c = w.ranks[0]
    model, ref = make(), make()
    ddp = FlexTreeDDP(model, c, bucket_bytes=4096, sharded=True)
    opt = ShardedOptimizer(ddp, lambda ps: torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.0))
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    assert all(c.in_heap(p.data) for p in model.parameters())
    x, y = torch.randn(16, 24, device=DEV), torch.randn(16, 7, device=DEV)
    for _ in range(3):
        opt.zero_grad()
        nn.functional.mse_loss(ddp(x), y).backward()
        opt.step()
        ropt.zero_grad()
        nn.functional.mse_loss(ref(x), y).backward()
        ropt.step()
    torch.cuda.synchronize()
    for p, r in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, r, atol=1e-6, rtol=1e-5)
    total = sum(p.numel() for p in ref.parameters())
    assert opt.state_elements() >= 2 * total
    opt.release()
    ddp.release()
    assert not any(c.in_heap(p.data) for p in model.parameters())
    w.close()


def test_auto_goes_through_the_native_policy_and_counts_the_algorithm():
    """algo="auto" leaves the choice to the native policy inside ft_allreduce: what choose() reports for a size is
    what the usage counters show afterwards; a device tensor larger than one staging slot is split natively."""
    w = LocalWorld(1, heap_bytes=1 << 20, staging_bytes=1 << 16)
    c = w.ranks[0]
    name, shape = c.choose(1 << 20, False, torch.float32)
    assert name in ("staged", "oneshot", "ll", "push") and P.validate_shape(1, shape) == ""
    big = torch.ones(100_000, device=DEV)        # 400 kB > the 64 KiB slot; world 1 copies, so the data must survive
    out = torch.empty_like(big)
    c.all_reduce(big, out=out)
    torch.cuda.synchronize()
    assert bool((out == 1).all())
    w.close()


def test_bounds_checked_build_runs_correct_plans_without_a_report():
    """The debugging build (-DFT_BOUNDS, lib/libflextree_bounds.so, FT_LIB=bounds): emulated worlds over tree, lonely,
    ring, one-shot, low-latency and reduce + push paths give the right sums and no kernel reports a range outside
    the heap.  Runs in a child process, since one process loads one build of the library."""
    import os
    import subprocess
    import sys
    from allreduce_over_mpi_b200.build import BOUNDS_LIB, NVCC
    if not BOUNDS_LIB.exists() and not os.path.exists(NVCC):
        pytest.skip("no bounds-checked build and no nvcc to make one")
    code = r"""
import torch
from allreduce_over_mpi_b200._lib import lib
from allreduce_over_mpi_b200.parallel.comm import LocalWorld
assert lib().ft_bounds_build() == 1
for world, shape in ((4, "2*2"), (5, "2*2+1"), (6, "ring6"), (8, "2*4"), (3, "3")):
    w = LocalWorld(world, heap_bytes=4 << 20, staging_bytes=1 << 20)
    for algo, heap in (("staged", True), ("staged", False), ("oneshot", False), ("ll", False), ("push", True)):
        for count in (5, 4099, 200_003):
            if algo == "ll" and count * 4 > (256 << 10):
                continue
            xs = []
            for r in range(world):
                if heap:
                    w.ranks[r].free_all()
                    t = w.ranks[r].alloc(count, torch.float32)
                else:
                    t = torch.empty(count, device="cuda:0")
                t.fill_(float(r + 1))
                xs.append(t)
            w.all_reduce(xs, shape=shape if algo == "staged" else None, algo=algo)
            torch.cuda.synchronize()
            want = world * (world + 1) / 2
            assert all(bool((x == want).all()) for x in xs), (world, shape, algo, count)
            for c in w.ranks:
                s = c.status()
                assert s["code"] == 0, (world, shape, algo, count, s)
    w.close()
print("BOUNDS-OK")
"""
    env = dict(os.environ, FT_LIB="bounds")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=root, timeout=900)
    assert r.returncode == 0 and "BOUNDS-OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
