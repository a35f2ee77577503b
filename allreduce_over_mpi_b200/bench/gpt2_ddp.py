"""GPT-2 small data-parallel training step: FlexTree gradient all-reduce vs NCCL DDP.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29512 \
        -m allreduce_over_mpi_b200.bench.gpt2_ddp --impl flextree nccl hook --steps 20 --warmup 5

Configuration: 12 layers, d_model 768, 12 heads, vocabulary 50257, sequence 1024, micro-batch 8
per GPU, bf16 parameters and gradients, random-init weights, random token ids, 25 MB gradient
buckets, fused AdamW.  ``flextree``: FlexTreeDDP (buckets in the symmetric heap, all-reduce on a
side stream overlapped with backward); ``hook``: torch DDP with the FlexTree comm hook;
``nccl``: torch DDP with NCCL.  Per step the token ids come from pinned host memory and the loss
is read back.  Time = max over ranks of a CUDA-event interval around the timed steps.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from ..models.gpt2 import GPT2, GPT2Config
from ..parallel.comm import FlexTreeComm
from ..parallel.ddp import FlexTreeDDP, HookState, flextree_allreduce_hook
from .allreduce import init_dist


def run(impl: str, a, rank: int, world: int, dev, comm) -> dict:
    torch.manual_seed(1234)
    cfg = GPT2Config.small() if not a.tiny else GPT2Config.tiny()
    model = GPT2(cfg).to(dev).to(torch.bfloat16)
    comm.free_all()   # every implementation starts from an empty symmetric heap
    sharded = None
    if impl == "flextree":
        ddp = FlexTreeDDP(model, comm, bucket_bytes=a.bucket_mb << 20)
        fwd, zero = ddp, ddp.zero_grad
    elif impl == "sharded":   # gradients reduce-scattered, AdamW state and update on this rank's blocks, parameters all-gathered
        from ..parallel.zero import ShardedOptimizer
        ddp = FlexTreeDDP(model, comm, bucket_bytes=a.bucket_mb << 20, sharded=True)
        sharded = ShardedOptimizer(ddp, lambda ps: torch.optim.AdamW(ps, lr=1e-4, fused=True))
        fwd, zero = ddp, ddp.zero_grad
    else:
        from torch.nn.parallel import DistributedDataParallel as DDP
        ddp = DDP(model, device_ids=[dev.index], bucket_cap_mb=a.bucket_mb, gradient_as_bucket_view=True) if world > 1 else model
        if impl == "hook" and world > 1:
            ddp.register_comm_hook(HookState(comm), flextree_allreduce_hook)
        fwd = ddp
        zero = lambda: model.zero_grad(set_to_none=False)  # noqa: E731
    opt = sharded if sharded is not None else torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    B, T = a.batch, min(a.seq, cfg.n_ctx)
    g = torch.Generator().manual_seed(100 + rank)
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g).pin_memory() for _ in range(4)]
    tok = torch.empty((B, T + 1), dtype=torch.long, device=dev)
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
    losses = []

    def step(i):
        tok.copy_(host_tokens[i % 4], non_blocking=True)
        zero()
        loss = fwd(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        loss_host.copy_(loss.detach(), non_blocking=True)

    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(a.steps):
        step(i)
        if i % 5 == 4:
            torch.cuda.current_stream().synchronize()
            losses.append(loss_host.item())
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / a.steps
    if comm is not None:
        comm.check()
    # parameters must agree across ranks after training
    chk = torch.stack([p.detach().float().sum() for p in model.parameters()]).sum().reshape(1)
    lo, hi = chk.clone(), chk.clone()
    if world > 1:
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    row = {"bench": "gpt2_ddp", "impl": impl, "world": world, "ms_per_step": round(ms, 3),
           "tokens_per_s": round(world * B * T / (ms * 1e-3), 1), "loss_last": losses[-1] if losses else None,
           "params_in_sync": bool(abs(lo.item() - hi.item()) <= 1e-3 * max(1.0, abs(hi.item()))),
           "model_params": model.num_params(), "batch_per_gpu": B, "seq": T, "bucket_mb": a.bucket_mb,
           "h2d_bytes_per_step": tok.numel() * 8, "d2h_bytes_per_step": 4}
    if sharded is not None:
        row["optimizer_state_elements_this_rank"] = sharded.state_elements()
    del opt, ddp, model
    torch.cuda.empty_cache()
    return row


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--impl", nargs="+", default=["flextree", "nccl"], choices=["flextree", "nccl", "hook", "sharded"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--lanes", type=int, default=0, help="cap on CTAs of the all-reduce kernel while it overlaps backward")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--repeats", type=int, default=1, help="run the whole list of implementations this many times")
    ap.add_argument("--clock-gpu", type=int, default=0, help="physical GPU index the clock sampler watches (0: this rank's device)")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank, world, local = init_dist()
    dev = torch.device("cuda", local)
    comm = FlexTreeComm(heap_bytes=1 << 30, staging_bytes=64 << 20)
    if a.lanes:
        comm.set_max_lanes(a.lanes)
    rows = []
    from ..utils import ClockSampler
    for rep in range(a.repeats):
        for impl in a.impl:
            sampler = ClockSampler(gpu_index=a.clock_gpu or torch.cuda.current_device()).start() if rank == 0 else None
            row = run(impl, a, rank, world, dev, comm)
            row["repeat"] = rep
            if sampler is not None:
                row["clocks"] = sampler.stop()   # SM clock under load and throttle reasons during this run (read-only sampling)
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
                if a.out:
                    with open(a.out, "a") as f:
                        f.write(json.dumps(row) + "\n")
    comm.close()
    if world > 1:
        dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
