"""Data-parallel gradient all-reduce through FlexTree, overlapped with backward.

Two integrations:

* :class:`FlexTreeDDP` - a DDP-style wrapper that owns the gradient storage.  Gradients live
  in flat buckets (25 MB by default) allocated *inside the symmetric heap*, every parameter's
  ``.grad`` is a view into its bucket, and as soon as the last gradient of a bucket has been
  accumulated the bucket is all-reduced in place on a side stream (zero copy, averaging fused
  into the kernel) while backward continues on the main stream.  With ``sharded=True`` the bucket
  is only reduce-scattered; ``parallel/zero.py`` builds the optimizer with split state on that.
* :func:`flextree_allreduce_hook` - a communication hook for ``torch.nn.parallel.
  DistributedDataParallel.register_comm_hook``; DDP keeps its own buckets, which are staged
  through the communicator's slots.

The reference has no trainer: its benchmark calls the all-reduce in a loop
(allreduce_over_mpi/benchmark.cpp:155-182).  This module is what connects the collective to
a training step.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Iterable

import torch
import torch.nn as nn


@dataclass
class Bucket:
    params: list = field(default_factory=list)
    offsets: list = field(default_factory=list)   # element offsets inside the flat buffer
    numel: int = 0
    dtype: torch.dtype = torch.float32
    flat: torch.Tensor | None = None
    pending: int = 0
    owned: list = field(default_factory=list)     # sharded mode: views of the blocks of `flat` this rank holds reduced


def build_buckets(params: Iterable[nn.Parameter], bucket_bytes: int = 25 << 20, align_elems: int = 64) -> list[Bucket]:
    """Assign parameters to buckets in reverse order (the order gradients become ready), one dtype
    per bucket, each parameter's slice aligned to ``align_elems`` elements."""
    buckets: list[Bucket] = []
    cur: dict[torch.dtype, Bucket] = {}
    for p in reversed([p for p in params if p.requires_grad]):
        b = cur.get(p.dtype)
        es = p.element_size()
        if b is None or (b.numel and (b.numel + p.numel()) * es > bucket_bytes):
            b = Bucket(dtype=p.dtype)
            cur[p.dtype] = b
            buckets.append(b)
        b.params.append(p)
        b.offsets.append(b.numel)
        b.numel += -(-p.numel() // align_elems) * align_elems
    return buckets


class FlexTreeDDP(nn.Module):
    """Wrap ``module`` for data-parallel training over ``comm`` (a FlexTreeComm or any object with
    ``alloc``, ``all_reduce``, ``world`` and ``device``)."""

    def __init__(self, module: nn.Module, comm, bucket_bytes: int = 25 << 20, shape=None, algo: str = "auto",
                 broadcast_from: int | None = 0, stream: torch.cuda.Stream | None = None, sharded: bool = False):
        """``sharded=True``: a bucket is only reduce-scattered (the first half of the all-reduce): afterwards each
        rank holds the averaged gradient of ITS blocks of the bucket (``Bucket.owned``) and partial sums elsewhere.
        That is the gradient side of an optimizer whose state is split over the ranks
        (:class:`~allreduce_over_mpi_b200.parallel.zero.ShardedOptimizer`)."""
        super().__init__()
        self.module = module
        self.comm = comm
        self.shape, self.algo = shape, algo
        self.sharded = sharded
        self.buckets = build_buckets(module.parameters(), bucket_bytes)
        self._bucket_of: dict[int, tuple[Bucket, int]] = {}
        on_gpu = torch.cuda.is_available() and getattr(comm, "device", torch.device("cpu")).type == "cuda"
        self.stream = stream or (torch.cuda.Stream(device=comm.device) if on_gpu else None)
        self._callback_queued = False
        self._sync = True
        self._hooks: list = []
        self.launched = 0
        for b in self.buckets:
            b.flat = comm.alloc(b.numel, b.dtype)
            b.flat.zero_()
            for p, off in zip(b.params, b.offsets):
                p.grad = b.flat[off:off + p.numel()].view_as(p)
                self._bucket_of[id(p)] = (b, off)
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
            b.pending = len(b.params)
        if broadcast_from is not None and comm.world > 1:
            self._sync_parameters(broadcast_from)

    def _sync_parameters(self, src: int):
        """Make every rank start from rank ``src``'s weights: zero everywhere else, then sum."""
        with torch.no_grad():
            for p in list(self.module.parameters()) + list(self.module.buffers()):
                if not p.is_floating_point():
                    continue
                if self.comm.rank != src:
                    p.zero_()
                self.comm.all_reduce(p.data, shape=self.shape)
        if self.stream is not None:
            torch.cuda.synchronize(self.comm.device)

    def forward(self, *args, **kwargs):
        # A backward that raised never reached _finish(): its half-counted buckets and the queued-callback mark
        # must not leak into the next step, where buckets would launch early or the side stream never be joined.
        if self._callback_queued or any(b.pending != len(b.params) for b in self.buckets):
            self._callback_queued = False
            for b in self.buckets:
                b.pending = len(b.params)
            if self.stream is not None:
                torch.cuda.current_stream(self.comm.device).wait_stream(self.stream)
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context only accumulate into the buckets (gradient accumulation);
        the first backward after it reduces the accumulated sums.  Every rank must use it alike."""
        prev, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = prev

    # -- backward-time machinery
    def _on_grad(self, p: nn.Parameter):
        b, off = self._bucket_of[id(p)]
        if p.grad.data_ptr() != b.flat.data_ptr() + off * p.element_size():
            # something replaced .grad (e.g. zero_grad(set_to_none=True)): fold it back into the bucket
            view = b.flat[off:off + p.numel()].view_as(p)
            view.copy_(p.grad)
            p.grad = view
        if not self._sync:
            return
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish)
        b.pending -= 1
        if b.pending == 0:
            self._launch(b)

    def _reduce(self, b: Bucket):
        if self.sharded:
            b.owned = self.comm.reduce_scatter(b.flat, op="avg", shape=self.shape)
        else:
            self.comm.all_reduce(b.flat, op="avg", shape=self.shape, algo=self.algo)

    def _launch(self, b: Bucket):
        self.launched += 1
        if self.stream is None:
            self._reduce(b)
            return
        self.stream.wait_stream(torch.cuda.current_stream(self.comm.device))
        with torch.cuda.stream(self.stream):
            self._reduce(b)

    def _finish(self):
        """End of backward: flush buckets only part of whose parameters got a gradient, join the side stream.
        A bucket none of whose parameters got a gradient is left alone, which is safe only when every rank has
        the same unused parameters (the rule torch DDP states for find_unused_parameters=False)."""
        for b in self.buckets:
            if 0 < b.pending < len(b.params):
                self._launch(b)
            b.pending = len(b.params)
        if self.stream is not None:
            torch.cuda.current_stream(self.comm.device).wait_stream(self.stream)
        self._callback_queued = False

    def release(self):
        """Detach the gradients from the symmetric heap and give the buckets back to the communicator (when it
        has ``free``).  The wrapper must not be used afterwards; every rank has to call this at the same point."""
        if self.stream is not None:
            torch.cuda.current_stream(self.comm.device).wait_stream(self.stream)
            torch.cuda.synchronize(self.comm.device)
        for h in self._hooks:
            h.remove()
        self._hooks = []
        for b in self.buckets:
            for p in b.params:
                p.grad = None
        free = getattr(self.comm, "free", None)
        for b in reversed(self.buckets):
            if free is not None and b.flat is not None:
                free(b.flat)
            b.flat = None
        self.buckets = []

    def zero_grad(self, set_to_none: bool = False):
        """Gradients are views of the symmetric buckets; they are zeroed in place, never released."""
        for b in self.buckets:
            b.flat.zero_()


# ---- torch DDP communication hook ----------------------------------------------------------
class HookState:
    """State of :func:`flextree_allreduce_hook`.  With ``mirror=True`` (default) every DDP bucket gets
    a twin in the symmetric heap: the bucket is copied there, reduced in place with the fastest
    algorithm for heap tensors (NVLS where available) and copied back - two local copies at HBM
    speed instead of a slower all-reduce through the staging slots."""

    def __init__(self, comm, shape=None, algo: str = "auto", mirror: bool = True):
        self.comm, self.shape, self.algo, self.mirror = comm, shape, algo, mirror
        self.stream = torch.cuda.Stream(device=comm.device)
        self.calls = 0
        self.twins: dict = {}

    def twin(self, bucket, buf: torch.Tensor):
        key = (bucket.index(), buf.numel(), buf.dtype)
        t = self.twins.get(key)
        if t is None:
            try:
                t = self.comm.alloc(buf.numel(), buf.dtype)
            except MemoryError:
                t = False   # heap exhausted: this bucket goes through the staging slots
            self.twins[key] = t
        return t


    def release(self):
        """Give the heap twins back (after the last backward has finished; same point on every rank)."""
        torch.cuda.synchronize(self.comm.device)
        for t in reversed(list(self.twins.values())):
            if t is not False:
                self.comm.free(t)
        self.twins = {}


def flextree_allreduce_hook(state, bucket):
    """``ddp.register_comm_hook(HookState(comm), flextree_allreduce_hook)``: average the bucket with
    FlexTree on a side stream and hand DDP a future that is complete in stream order."""
    buf = bucket.buffer()
    dev = state.comm.device
    state.calls += 1
    state.stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(state.stream):
        twin = state.twin(bucket, buf) if state.mirror else False
        if twin is not False:
            twin.copy_(buf)
            state.comm.all_reduce(twin, op="avg", shape=state.shape, algo=state.algo)
            buf.copy_(twin)
        else:
            state.comm.all_reduce(buf, op="avg", shape=state.shape, algo=state.algo)
        fut: torch.futures.Future = torch.futures.Future(devices=[dev])
        fut.set_result(buf)
    return fut


# torch validates the hook's signature with real annotation objects (this module postpones
# annotation evaluation, so they are attached here)
flextree_allreduce_hook.__annotations__ = {"return": torch.futures.Future[torch.Tensor]}
try:
    import torch.distributed as _dist
    flextree_allreduce_hook.__annotations__["bucket"] = _dist.GradBucket
except (ImportError, AttributeError):  # torch built without distributed support
    pass
