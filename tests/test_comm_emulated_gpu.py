"""Collective kernels on ONE GPU: the ranks of a world are emulated by launching each stage of
the plan rank after rank on one stream with the rendezvous switched off, so no kernel ever
waits on another.  Results are compared with the CPU snapshot executor (same plan, same block
geometry) and with an fp64 sum."""
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


SHAPES = ["2", "3", "4", "2*2", "5", "2*2+1", "6", "2*3", "3*2", "2*2+2", "7", "2*3+1", "3*2+1", "8", "2*4", "4*2",
          "2*2*2", "ring4", "ring8", "2*3+2", "3*3", "2*2*2+1", "2*2*3"]


@pytest.mark.parametrize("text", SHAPES)
def test_staged_shapes_fp32_staging_mode(text):
    shape = Shape.parse(text)
    w = LocalWorld(shape.world, heap_bytes=1 << 20, staging_bytes=4 << 20)
    for count in (1, 35, 4099, 300_000):
        host = inputs(shape.world, count, torch.float32)
        want = torch.stack(host).double().sum(0)
        dev = [h.to(DEV) for h in host]
        w.all_reduce(dev, shape=shape)
        torch.cuda.synchronize()
        for r in range(shape.world):
            assert torch.allclose(dev[r].double().cpu(), want, atol=1e-5), (text, count, r)
        assert all(torch.equal(d, dev[0]) for d in dev)  # one reducer per block: bit-identical everywhere
    w.close()


@pytest.mark.parametrize("text", ["4", "2*2+1", "2*4", "2*2*2", "ring5", "3*2+1"])
def test_staged_in_heap_zero_copy(text):
    shape = Shape.parse(text)
    w = LocalWorld(shape.world, heap_bytes=8 << 20, staging_bytes=1 << 16)
    for count in (1000, 777_777):
        host = inputs(shape.world, count, torch.float32, seed=3)
        want = torch.stack(host).double().sum(0)
        dev = []
        for r, c in enumerate(w.ranks):
            t = c.alloc(count, torch.float32)
            assert c.in_heap(t)
            t.copy_(host[r])
            dev.append(t)
        w.all_reduce(dev, shape=shape)
        torch.cuda.synchronize()
        for r in range(shape.world):
            assert torch.allclose(dev[r].double().cpu(), want, atol=1e-5), (text, count, r)
        for c in w.ranks:
            c.free_all()
    w.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int32, torch.int64,
                                   torch.uint8, torch.int8, torch.int16])
def test_dtypes_match_cpu_executor(dtype):
    shape = Shape.parse("2*3+1")
    w = LocalWorld(7, heap_bytes=1 << 20, staging_bytes=1 << 20)
    for count in (37, 10_001):
        host = inputs(7, count, dtype, seed=5)
        dev = [h.to(DEV) for h in host]
        w.all_reduce(dev, shape=shape)
        torch.cuda.synchronize()
        # the CPU executor with the SAME block size performs the same additions in the same order
        es = host[0].element_size()
        per = 16 // es
        block = -(-count // 7)
        block = -(-block // per) * per
        P.run_plan_snapshot(shape, host, block_elems=block)
        for r in range(7):
            if dtype.is_floating_point:
                assert torch.allclose(dev[r].cpu().double(), host[r].double(), atol=tol(dtype)), (dtype, count, r)
            else:
                assert torch.equal(dev[r].cpu(), host[r]), (dtype, count, r)
    w.close()


def test_band_and_unsupported():
    w = LocalWorld(4, heap_bytes=1 << 20, staging_bytes=1 << 20)
    host = [torch.randint(0, 2 ** 31 - 1, (5000,), dtype=torch.int32) for _ in range(4)]
    dev = [h.to(DEV) for h in host]
    w.all_reduce(dev, op="band", shape="2*2")
    torch.cuda.synchronize()
    assert torch.equal(dev[2].cpu(), host[0] & host[1] & host[2] & host[3])
    with pytest.raises(Exception, match="not supported"):
        w.all_reduce([torch.rand(8, device=DEV) for _ in range(4)], op="band", shape="4")
    with pytest.raises(Exception, match="invalid FT_TOPO"):
        w.all_reduce([torch.rand(8, device=DEV) for _ in range(4)], shape="3*2")
    w.close()


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_oneshot(world, dtype):
    w = LocalWorld(world, heap_bytes=1 << 20, staging_bytes=1 << 20)
    for it, count in enumerate((1, 9, 4096, 100_001)):
        host = inputs(world, count, dtype, seed=it)
        want = torch.stack(host).double().sum(0)
        dev = [h.to(DEV) for h in host]
        w.all_reduce(dev, algo="oneshot")     # successive calls alternate between the two staging slots
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.allclose(dev[r].double().cpu(), want, atol=tol(dtype) * 2), (world, count, r)
        assert all(torch.equal(d, dev[0]) for d in dev)
    w.close()


@pytest.mark.parametrize("world", [2, 5, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_low_latency_push(world, dtype):
    w = LocalWorld(world, heap_bytes=1 << 20, staging_bytes=1 << 20)
    for it, count in enumerate((1, 3, 9, 1000, 65536, 77)):
        host = inputs(world, count, dtype, seed=20 + it)
        want = torch.stack(host).double().sum(0)
        dev = [h.to(DEV) for h in host]
        w.all_reduce(dev, algo="ll")       # successive calls alternate between the two receive areas
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.allclose(dev[r].double().cpu(), want, atol=tol(dtype) * 2), (world, count, r)
        assert all(torch.equal(d, dev[0]) for d in dev)
    with pytest.raises(Exception, match="256 KiB"):
        w.all_reduce([torch.zeros(100_000, device=DEV) for _ in range(world)], algo="ll")
    w.close()


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
def test_reduce_and_push(world, dtype):
    w = LocalWorld(world, heap_bytes=8 << 20, staging_bytes=1 << 16)
    for it, count in enumerate((1, 35, 4099, 500_001)):
        host = inputs(world, count, dtype, seed=40 + it)
        want = torch.stack(host).double().sum(0)
        dev = []
        for r, c in enumerate(w.ranks):
            t = c.alloc(count, dtype)
            t.copy_(host[r])
            dev.append(t)
        w.all_reduce(dev, algo="push")
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.allclose(dev[r].double().cpu(), want, atol=tol(dtype) * 2), (world, count, r)
        assert all(torch.equal(d, dev[0]) for d in dev)
        for c in w.ranks:
            c.free_all()
    with pytest.raises(Exception, match="symmetric heap"):
        w.all_reduce([torch.zeros(64, device=DEV) for _ in range(world)], algo="push")
    w.close()


def test_scale_and_out_of_place():
    w = LocalWorld(4, heap_bytes=1 << 20, staging_bytes=1 << 20)
    host = inputs(4, 12_345, torch.bfloat16, seed=9)
    want = (torch.stack(host).float().sum(0) / 4)
    src = [h.to(DEV) for h in host]
    dst = [torch.zeros_like(s) for s in src]
    w.all_reduce(src, op="avg", shape="2*2", outs=dst)
    torch.cuda.synchronize()
    for r in range(4):
        assert torch.equal(src[r].cpu(), host[r])           # inputs untouched
        assert torch.allclose(dst[r].float().cpu(), want, atol=2e-2)
    dst2 = [torch.zeros_like(s) for s in src]
    w.all_reduce(src, op="avg", algo="oneshot", outs=dst2)
    torch.cuda.synchronize()
    assert torch.allclose(dst2[1].float().cpu(), want, atol=2e-2)
    w.close()


def test_unaligned_user_tensors():
    w = LocalWorld(3, heap_bytes=1 << 20, staging_bytes=1 << 20)
    host = inputs(3, 5001, torch.float32, seed=11)
    want = torch.stack(host).double().sum(0)
    base = [torch.zeros(5010, device=DEV) for _ in range(3)]
    views = [b[1 + r:1 + r + 5001] for r, b in enumerate(base)]   # element-aligned only
    for v, h in zip(views, host):
        v.copy_(h)
    w.all_reduce(views, shape="3")
    torch.cuda.synchronize()
    for r in range(3):
        assert torch.allclose(views[r].double().cpu(), want, atol=1e-5)
        assert base[r][:1 + r].abs().sum() == 0 and base[r][1 + r + 5001:].abs().sum() == 0
    w.close()


def test_world_of_one_and_bounded_wait():
    w = LocalWorld(1, heap_bytes=1 << 20, staging_bytes=1 << 20)
    c = w.ranks[0]
    x = torch.rand(1000, device=DEV)
    y = x.clone()
    c.all_reduce(y)
    assert torch.equal(x, y)
    z = torch.empty_like(x)
    c.all_reduce(x, out=z, op="avg")
    assert torch.allclose(z, x)
    # a wait that nothing will ever satisfy comes back with a timeout status, the context stays usable
    assert c.status()["code"] == 0
    c.wait_probe(peer=0, timeout_ms=2.0)
    with pytest.raises(Exception, match="timeout"):
        c.check()
    assert c.status()["code"] == 0
    c.all_reduce(y)
    torch.cuda.synchronize()
    w.close()


@pytest.mark.parametrize("text", SHAPES)
def test_plans_on_tagged_words(text):
    """Every shape with the low-latency protocol (ll_tree_allreduce_kernel): each edge of a stage is a push of tagged
    8-byte words, no rendezvous.  Same sums as the staged kernel bit for bit (same plan, same summation order), out of
    place and in place, odd lengths, several calls in a row (the two receive areas alternate), averaging fused."""
    shape = Shape.parse(text)
    n = shape.world
    w = LocalWorld(n, heap_bytes=1 << 20, staging_bytes=1 << 20)
    for dtype in (torch.float32, torch.bfloat16):
        for count in (1, 35, 4099, 30_001):
            host = inputs(n, count, dtype, seed=5)
            want = torch.stack(host).double().sum(0)
            ref = [h.to(DEV) for h in host]
            w.all_reduce(ref, shape=shape, algo="staged")
            src = [h.to(DEV) for h in host]
            out = [torch.full_like(s, float("nan")) for s in src]
            w.all_reduce(src, shape=shape, algo="ll", outs=out)      # out of place
            inp = [h.to(DEV) for h in host]
            w.all_reduce(inp, shape=shape, algo="ll")                # in place, next call parity
            torch.cuda.synchronize()
            for r in range(n):
                assert torch.allclose(out[r].double().cpu(), want, atol=tol(dtype) * n), (text, dtype, count, r)
                assert torch.equal(out[r], ref[r]) and torch.equal(inp[r], ref[r]), (text, dtype, count, r)
                assert torch.equal(src[r].cpu(), host[r])            # the input of an out-of-place call is untouched
    avg = [torch.full((1000,), float(r + 1), device=DEV) for r in range(n)]
    w.all_reduce(avg, shape=shape, algo="ll", op="avg")
    torch.cuda.synchronize()
    assert all(torch.allclose(a, torch.full_like(a, (n + 1) / 2), atol=1e-6) for a in avg)
    for c in w.ranks:
        assert c.status()["code"] == 0
    w.close()
