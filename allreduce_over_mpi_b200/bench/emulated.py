"""Collective kernels on ONE GPU with the ranks emulated (stage after stage, rank after rank, in
stream order; no kernel waits on another).  Peer loads then hit this GPU's own HBM, so the numbers
show what the kernels do when the wires are not the limit - the reduce/HBM side of the roofline -
and the run is small and self-terminating, suitable for a profiler capture of a single kernel:

    python -m allreduce_over_mpi_b200.bench.emulated --world 8 --bytes 268435456 --shape 8 --algo staged
    ncu --set full --clock-control none -k regex:staged_allreduce -s 8 -c 2 -o prof \
        python -m allreduce_over_mpi_b200.bench.emulated --world 8 --bytes 268435456 --shape 8 --iters 1

With --algo staged the per-stage device time is printed (publish, stage 0, ...), the counterpart of
the reference's SHOW_TIME phase log.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..parallel import planner
from ..parallel.comm import LocalWorld
from ..parallel.planner import Shape


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--shape", default=None)
    ap.add_argument("--algo", default="staged", choices=["staged", "oneshot", "ll", "push"])
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    dtype = getattr(torch, a.dtype)
    es = torch.empty((), dtype=dtype).element_size()
    count = a.bytes // es
    shape = Shape.parse(a.shape) if a.shape else Shape.flat(a.world)
    in_heap = a.algo in ("staged", "push")
    heap = a.bytes + (1 << 20) if in_heap else 1 << 20
    w = LocalWorld(a.world, heap_bytes=heap, staging_bytes=max(a.bytes, 1 << 20) if not in_heap else 1 << 20)
    g = torch.Generator(device="cuda").manual_seed(7)
    if in_heap:
        bufs = [c.alloc(count, dtype) for c in w.ranks]
    else:
        bufs = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(a.world)]
    for b in bufs:
        b.copy_((torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype))
    want = torch.stack([b.double() for b in bufs]).sum(0)
    w.all_reduce(bufs, shape=shape, algo=a.algo)
    torch.cuda.synchronize()
    err = (bufs[-1].double() - want).abs().max().item()
    row = {"bench": "emulated", "algo": a.algo, "world": a.world, "shape": str(shape), "bytes": a.bytes, "dtype": a.dtype,
           "max_abs_err": err}
    if a.algo == "staged" and a.iters > 0:
        ms = w.profile_stages(bufs, shape, iters=a.iters)
        row["stage_ms"] = [round(x, 4) for x in ms]
        # bytes each stage moves through HBM on this one GPU: all ranks' reads + writes
        plan = planner.plan_json(a.world, shape)
        per_stage = []
        for s in range(plan["stages"]):
            blocks = sum(len(p[2]) + (2 if p[1] else 1) for r in range(a.world) for p in plan["ranks"][r][s]["pulls"])
            per_stage.append(blocks * a.bytes / a.world)
        row["stage_GBps"] = [round(b / (t * 1e-3) / 1e9, 1) if t > 0 else None for b, t in zip(per_stage, ms[1:])]
    elif a.iters > 0:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.iters):
            w.all_reduce(bufs, algo=a.algo)
        e.record()
        e.synchronize()
        row["ms_all_ranks"] = round(s.elapsed_time(e) / a.iters, 4)
    print(json.dumps(row), flush=True)
    w.close()
    return 0 if err < (1e-3 if dtype == torch.float32 else 1.0) else 1


if __name__ == "__main__":
    sys.exit(main())
