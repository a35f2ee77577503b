"""Bucketing and backward-time scheduling of FlexTreeDDP on CPU with a stand-in communicator
(the real one needs GPUs).  world = 3 ranks are simulated by running the wrapper three times
and averaging inside the fake all_reduce."""
import torch
import torch.nn as nn

from allreduce_over_mpi_b200.models.gpt2 import GPT2, GPT2Config
from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP, build_buckets


class FakeComm:
    world, rank = 1, 0
    device = torch.device("cpu")

    def __init__(self):
        self.calls = []

    def alloc(self, shape, dtype=torch.float32):
        return torch.zeros(shape, dtype=dtype)

    def all_reduce(self, t, op="sum", shape=None, algo="auto", **kw):
        self.calls.append((t.numel(), op))
        return t


def test_buckets_cover_all_params_in_reverse_order():
    m = GPT2(GPT2Config.tiny())
    buckets = build_buckets(m.parameters(), bucket_bytes=64 << 10)
    ps = [p for p in m.parameters() if p.requires_grad]
    seen = [id(p) for b in buckets for p in b.params]
    assert seen == [id(p) for p in reversed(ps)]
    assert len(buckets) > 2
    for b in buckets:
        assert all(o % 64 == 0 for o in b.offsets)
        assert b.numel * 4 <= (64 << 10) or len(b.params) == 1
        assert b.numel >= sum(p.numel() for p in b.params)


def test_grads_match_plain_backward_and_every_bucket_fires_once():
    torch.manual_seed(0)
    ref = GPT2(GPT2Config.tiny())
    ddp_model = GPT2(GPT2Config.tiny())
    ddp_model.load_state_dict(ref.state_dict())
    comm = FakeComm()
    ddp = FlexTreeDDP(ddp_model, comm, bucket_bytes=64 << 10)
    x = torch.randint(0, 512, (2, 64))
    for step in range(2):
        ref.zero_grad()
        ddp.zero_grad()
        comm.calls.clear()
        ref(x, x).backward()
        ddp(x, x).backward()
        assert len(comm.calls) == len(ddp.buckets)
        assert all(op == "avg" for _, op in comm.calls)
        for (n1, p1), (n2, p2) in zip(ref.named_parameters(), ddp_model.named_parameters()):
            assert torch.allclose(p1.grad, p2.grad, atol=1e-6), n1
        # gradients are views of the flat buckets (zero copy into the collective)
        b = ddp.buckets[0]
        assert b.params[0].grad.data_ptr() == b.flat.data_ptr()


def test_unused_parameters_still_flush():
    class Two(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(8, 8), nn.Linear(8, 8)

        def forward(self, x):
            return self.a(x).sum()   # self.b gets no gradient

    comm = FakeComm()
    ddp = FlexTreeDDP(Two(), comm, bucket_bytes=1 << 20)
    ddp(torch.rand(4, 8)).backward()
    assert len(comm.calls) == 1      # the single bucket is flushed at the end of backward
    ddp(torch.rand(4, 8)).backward()
    assert len(comm.calls) == 2


def test_no_sync_accumulates_then_reduces_once():
    torch.manual_seed(1)
    ref = nn.Sequential(nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 4))
    mod = nn.Sequential(nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 4))
    mod.load_state_dict(ref.state_dict())
    comm = FakeComm()
    ddp = FlexTreeDDP(mod, comm, bucket_bytes=1 << 20)
    xs = [torch.rand(3, 16) for _ in range(3)]
    with ddp.no_sync():
        for x in xs[:2]:
            ddp(x).sum().backward()
    assert comm.calls == []                      # nothing was sent while accumulating
    ddp(xs[2]).sum().backward()
    assert len(comm.calls) == len(ddp.buckets)   # the accumulated sums go out once
    for x in xs:
        ref(x).sum().backward()
    for p1, p2 in zip(ref.parameters(), mod.parameters()):
        assert torch.allclose(p1.grad, p2.grad, atol=1e-6)


def test_release_returns_the_buckets():
    class Comm(FakeComm):
        def __init__(self):
            super().__init__()
            self.live = []

        def alloc(self, shape, dtype=torch.float32):
            t = super().alloc(shape, dtype)
            self.live.append(t.data_ptr())
            return t

        def free(self, t):
            self.live.remove(t.data_ptr())

    comm = Comm()
    model = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 2))
    ddp = FlexTreeDDP(model, comm, bucket_bytes=128)
    assert len(comm.live) == len(ddp.buckets) > 1
    ddp(torch.rand(3, 8)).sum().backward()
    ddp.release()
    assert comm.live == [] and all(p.grad is None for p in model.parameters()) and ddp.buckets == []
    model(torch.rand(3, 8)).sum().backward()      # the bare module trains on with ordinary gradients
    assert all(p.grad is not None for p in model.parameters())


def test_a_backward_that_raised_does_not_poison_the_next_step():
    """A backward that raises part-way leaves buckets half counted and the end-of-backward callback unrun; the next
    forward resets both, so the following step launches every bucket exactly once and gives the plain gradients."""
    torch.manual_seed(0)
    ref = GPT2(GPT2Config.tiny())
    model = GPT2(GPT2Config.tiny())
    model.load_state_dict(ref.state_dict())
    comm = FakeComm()
    ddp = FlexTreeDDP(model, comm, bucket_bytes=64 << 10)
    x = torch.randint(0, 512, (2, 64))
    # simulate the state a raising backward leaves behind
    ddp._callback_queued = True
    ddp.buckets[0].pending -= 1
    ddp.zero_grad()
    ref.zero_grad()
    comm.calls.clear()
    ref(x, x).backward()
    ddp(x, x).backward()
    assert len(comm.calls) == len(ddp.buckets)
    assert not ddp._callback_queued and all(b.pending == len(b.params) for b in ddp.buckets)
    for (n1, p1), (_, p2) in zip(ref.named_parameters(), model.named_parameters()):
        assert torch.allclose(p1.grad, p2.grad, atol=1e-6), n1
