"""Tiny end-to-end pass used by the repository's smoke check (one GPU)."""
from __future__ import annotations

import torch

from ..models.gpt2 import GPT2, GPT2Config
from .comm import LocalWorld
from .ddp import FlexTreeDDP


def smoke_comm_and_model(dev: torch.device) -> None:
    # four ranks emulated on this GPU: tree 2*2 and one-shot, checked against a plain sum
    w = LocalWorld(4, devices=[dev.index] * 4, heap_bytes=4 << 20, staging_bytes=1 << 20)
    xs = [torch.full((10_000,), float(r + 1), device=dev) for r in range(4)]
    w.all_reduce(xs, shape="2*2")
    ys = [torch.full((999,), float(r + 1), device=dev).bfloat16() for r in range(4)]
    w.all_reduce(ys, algo="oneshot")
    torch.cuda.synchronize(dev)
    assert all(bool((x == 10).all()) for x in xs) and all(bool((y == 10).all()) for y in ys)
    w.close()
    # one forward + backward + optimiser step of a 2-layer GPT-2 whose gradients live in the
    # communicator's symmetric heap and go through FlexTreeDDP (world of one rank)
    w1 = LocalWorld(1, devices=[dev.index], heap_bytes=16 << 20, staging_bytes=1 << 20)
    model = GPT2(GPT2Config.tiny()).to(dev).to(torch.bfloat16)
    ddp = FlexTreeDDP(model, w1.ranks[0], bucket_bytes=64 << 10)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    tok = torch.randint(0, 512, (2, 65), device=dev)
    loss = ddp(tok[:, :-1], tok[:, 1:])
    loss.backward()
    opt.step()
    torch.cuda.synchronize(dev)
    assert torch.isfinite(loss).item() and ddp.launched == len(ddp.buckets)
    w1.close()
