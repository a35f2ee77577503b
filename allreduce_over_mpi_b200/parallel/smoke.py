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
    # the low-latency push protocol, the flat reduce + push kernel (heap tensors) and a lonely layout, same world
    zs = [torch.full((777,), float(r + 1), device=dev) for r in range(4)]
    w.all_reduce(zs, algo="ll")
    ps = [w.ranks[r].alloc(4096, torch.bfloat16) for r in range(4)]
    for r, p in enumerate(ps):
        p.fill_(float(r + 1))
    w.all_reduce(ps, algo="push", op="avg")
    torch.cuda.synchronize(dev)
    assert all(bool((z == 10).all()) for z in zs) and all(bool((p == 2.5).all()) for p in ps)
    w.close()
    w5 = LocalWorld(5, devices=[dev.index] * 5, heap_bytes=1 << 20, staging_bytes=1 << 20)
    ls = [torch.full((1000,), float(r + 1), device=dev) for r in range(5)]
    w5.all_reduce(ls, shape="2*2+1")
    torch.cuda.synchronize(dev)
    assert all(bool((x == 15).all()) for x in ls)
    w5.close()
    # single-GPU n-way reduce: 8 bytes per thread (fp32, fan-in 4), 32-byte accesses, the scaled / casting kernel,
    # and the pipeline for operands in host memory
    from ..ops import HostReducePipeline, reduce_nway, reduce_nway_scaled
    fs = [torch.randn(1 << 16, device=dev) for _ in range(4)]
    want = torch.stack(fs).sum(0)
    assert torch.allclose(reduce_nway(fs), want, atol=1e-5)                  # 32-byte accesses (the default)
    assert torch.allclose(reduce_nway(fs, variant=24), want, atol=1e-5)      # 8 bytes per thread
    assert torch.allclose(reduce_nway(fs[:2], variant=13), fs[0] + fs[1], atol=1e-6)   # 16-byte vectors, persistent grid
    got = reduce_nway_scaled(fs, scale=0.25, out_dtype=torch.bfloat16)
    assert torch.allclose(got.float(), want * 0.25, atol=3e-2)
    hin = [f.cpu().pin_memory() for f in fs]
    hout = [torch.empty_like(hin[0]).pin_memory() for _ in range(2)]
    pipe = HostReducePipeline(device=dev, chunk_bytes=64 << 10, max_inputs=4, max_outputs=2)
    pipe.run(hin, [2, 4], hout)
    torch.cuda.synchronize(dev)
    assert torch.allclose(hout[1], want.cpu(), atol=1e-5) and torch.allclose(hout[0], (fs[0] + fs[1]).cpu(), atol=1e-6)
    pipe.close()
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
