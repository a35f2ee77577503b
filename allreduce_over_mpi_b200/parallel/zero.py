"""Optimizer with its state split over the ranks, on the two halves of the all-reduce.

An all-reduce is a reduce-scatter followed by an all-gather (allreduce_over_mpi/mpi_mod.hpp:1550-1596
and :1620-1644 are the reference's two loops).  A data-parallel step does not need both halves on the
gradients: after the reduce-scatter every rank holds the averaged gradient of ITS blocks, which is enough
to update ITS blocks of the parameters; the all-gather then distributes updated parameters instead of
gradients.  The wire carries the same bytes as one all-reduce, but the optimizer's state (two fp32
moments per parameter for Adam) and its arithmetic exist once per job instead of once per rank.

    ddp = FlexTreeDDP(model, comm, sharded=True)          # buckets are reduce-scattered during backward
    opt = ShardedOptimizer(ddp, lambda ps: torch.optim.AdamW(ps, lr=3e-4))
    loss(ddp(x)).backward(); opt.step(); opt.zero_grad()

Works on any communicator with ``alloc``, ``reduce_scatter`` and ``all_gather`` in place on its own tensors:
``FlexTreeComm`` (GPUs; from five ranks up the halves run through the switch with ``multimem``) and
``ProcWorld`` with a shared heap (CPU processes).
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch
import torch.nn as nn

from .ddp import FlexTreeDDP


class ShardedOptimizer:
    """Wraps ``make_optimizer`` (a callable from a parameter list to a ``torch.optim.Optimizer``) so that each
    rank updates only the blocks of every bucket it owns.

    Construction is collective: the module's parameters move into flat buffers of the communicator's heap (one
    per gradient bucket, same layout), and one reduce-scatter of the still empty gradient buckets tells every
    rank which element ranges are its own - the communicator's block arithmetic is not repeated here."""

    def __init__(self, ddp: FlexTreeDDP, make_optimizer: Callable[[Iterable[nn.Parameter]], torch.optim.Optimizer]):
        if not ddp.sharded:
            raise ValueError("needs FlexTreeDDP(..., sharded=True): gradients must be reduce-scattered, not all-reduced")
        self.ddp = ddp
        self.comm = ddp.comm
        self.param_flats: list[torch.Tensor] = []
        self.shards: list[nn.Parameter] = []
        self.ranges: list[list[tuple[int, int]]] = []     # per bucket: the element ranges [lo, hi) this rank owns
        for b in ddp.buckets:
            pflat = self.comm.alloc(b.numel, b.dtype)
            pflat.zero_()
            with torch.no_grad():
                for p, off in zip(b.params, b.offsets):
                    view = pflat[off:off + p.numel()].view_as(p)
                    view.copy_(p.data)
                    p.data = view
            self.param_flats.append(pflat)
            es = b.flat.element_size()
            owned = self.comm.reduce_scatter(b.flat, op="sum", shape=ddp.shape)      # zeros in, zeros out: only the views matter
            rng = []
            for v in owned:
                lo = (v.data_ptr() - b.flat.data_ptr()) // es
                if v.numel() == 0:
                    continue
                rng.append((lo, lo + v.numel()))
                shard = nn.Parameter(pflat[lo:lo + v.numel()], requires_grad=True)   # aliases the flat buffer: step() writes through
                shard.grad = b.flat[lo:lo + v.numel()]
                self.shards.append(shard)
            self.ranges.append(rng)
        self._sync()
        # a rank that owns nothing (more ranks than 16-byte vectors in a tiny model) still takes part in the collectives
        self.optimizer = make_optimizer(self.shards) if self.shards else None

    def _sync(self):
        if self.comm.device.type == "cuda":
            torch.cuda.synchronize(self.comm.device)

    @property
    def param_groups(self):
        return self.optimizer.param_groups if self.optimizer is not None else []

    def state_elements(self) -> int:
        """Elements of optimizer state this rank holds (for Adam: two per owned parameter element)."""
        if self.optimizer is None:
            return 0
        return sum(t.numel() for st in self.optimizer.state.values() for t in st.values() if torch.is_tensor(t))

    @torch.no_grad()
    def step(self):
        """Update the owned blocks from their averaged gradients, then all-gather the parameters.  Call after
        ``backward()`` has returned (the reduce-scatters have been joined to the current stream by then)."""
        if self.optimizer is not None:
            self.optimizer.step()
        for pflat in self.param_flats:
            self.comm.all_gather(pflat, shape=self.ddp.shape)

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float, eps: float = 1e-6) -> torch.Tensor:
        """Scale the owned gradient blocks so that the 2-norm of the WHOLE averaged gradient is at most ``max_norm``
        (what ``torch.nn.utils.clip_grad_norm_`` does for an unsplit gradient).  Every block has exactly one owner,
        so the squared norms of the shards add up to the squared global norm: one all-reduce of a single number.
        Call between ``backward()`` and :meth:`step`, on every rank.  Returns the global norm."""
        dev = self.comm.device
        sq = torch.zeros(1, dtype=torch.float32, device=dev)
        for shard in self.shards:
            sq += shard.grad.float().pow(2).sum()
        if self.comm.world > 1:
            self.comm.all_reduce(sq, op="sum")
        norm = sq.sqrt()
        scale = (max_norm / (norm + eps)).clamp(max=1.0)
        for shard in self.shards:
            shard.grad.mul_(scale.to(shard.grad.dtype))
        return norm[0]

    def zero_grad(self, set_to_none: bool = False):
        """The shards' gradients are views of the gradient buckets, which are zeroed in place."""
        self.ddp.zero_grad()

    def state_dict(self) -> dict:
        """This rank's part: the wrapped optimizer's state over its shards, and which ranges those are."""
        return {"ranges": self.ranges, "optimizer": self.optimizer.state_dict() if self.optimizer is not None else None}

    def load_state_dict(self, sd: dict):
        if sd["ranges"] != self.ranges:
            raise ValueError("state was saved for another world size, rank or bucket layout")
        if self.optimizer is not None:
            self.optimizer.load_state_dict(sd["optimizer"])

    def release(self):
        """Move the parameters back to ordinary memory and return the flat buffers to the communicator (collective,
        same point on every rank); the wrapper must not be used afterwards."""
        self._sync()
        with torch.no_grad():
            for b in self.ddp.buckets:
                for p in b.params:
                    p.data = p.data.clone()
        free = getattr(self.comm, "free", None)
        for pflat in reversed(self.param_flats):
            if free is not None:
                free(pflat)
        self.param_flats, self.shards, self.optimizer = [], [], None
