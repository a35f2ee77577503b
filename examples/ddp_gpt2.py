"""Minimal data-parallel training loop with FlexTree gradient all-reduce (one process per GPU):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 examples/ddp_gpt2.py [--sharded]

--sharded: the optimizer's state is split over the ranks (gradients reduce-scattered, parameters all-gathered).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from allreduce_over_mpi_b200.models.gpt2 import GPT2, GPT2Config  # noqa: E402
from allreduce_over_mpi_b200.parallel.comm import FlexTreeComm  # noqa: E402
from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP  # noqa: E402

local = int(os.environ.get("LOCAL_RANK", 0))
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))   # bootstrap only
comm = FlexTreeComm(heap_bytes=1 << 30)
model = GPT2(GPT2Config.small()).cuda().bfloat16()
if "--sharded" in sys.argv:
    from allreduce_over_mpi_b200.parallel.zero import ShardedOptimizer
    ddp = FlexTreeDDP(model, comm, sharded=True)   # buckets are only reduce-scattered: each rank gets its blocks' gradient
    opt = ShardedOptimizer(ddp, lambda ps: torch.optim.AdamW(ps, lr=3e-4, fused=True))   # 1/N of AdamW's state per rank
else:
    ddp = FlexTreeDDP(model, comm)             # gradients live in the symmetric heap, 25 MB buckets
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True)
for step in range(10):
    tok = torch.randint(0, 50257, (8, 1025), device="cuda")
    ddp.zero_grad()
    loss = ddp(tok[:, :-1], tok[:, 1:])
    loss.backward()                            # buckets are averaged on a side stream while backward continues
    opt.step()
    if dist.get_rank() == 0:
        print(f"step {step} loss {loss.item():.3f}")
comm.check()
comm.close()
dist.destroy_process_group()
