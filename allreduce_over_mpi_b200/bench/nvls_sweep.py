"""Sweep of the NVLS kernels' launch shape (threads per CTA, vectors in flight per thread, CTAs per launch,
instruction form, ownership stripes) on the GPUs of one NVSwitch box, next to NCCL on the same buffer.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29512 \
        -m allreduce_over_mpi_b200.bench.nvls_sweep --bytes 67108864 268435456 --dtype float32 \
        --threads 256 512 1024 --unroll 2 4 8 --lanes 0 32 64 96 --stripe 0 262144 --out nvls_sweep.jsonl

Timing as in bench/allreduce.py: CUDA events on the launching stream, L2 flushed between iterations, median
over iterations of the max over ranks.  One JSON line per configuration; ``--phases`` adds the reduce-scatter
and all-gather halves (multimem pass each) next to the staged peer-load halves and NCCL's.
"""
from __future__ import annotations

import argparse
import itertools
import json
import sys

import torch
import torch.distributed as dist

from .allreduce import busbw, fill, init_dist, make_comm, time_collective


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--bytes", type=int, nargs="+", default=[64 << 20, 256 << 20])
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--threads", type=int, nargs="+", default=[512])
    ap.add_argument("--unroll", type=int, nargs="+", default=[4])
    ap.add_argument("--weak", type=int, nargs="+", default=[0])
    ap.add_argument("--lanes", type=int, nargs="+", default=[0])
    ap.add_argument("--stripe", type=int, nargs="+", default=[0])
    ap.add_argument("--ctas-per-sm", type=int, nargs="+", default=[1])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--others", nargs="*", default=["push", "nccl"], help="also time these on the same buffer: push, staged, hybrid, nccl")
    ap.add_argument("--peer-lanes", type=int, nargs="+", default=[0], help="CTA caps tried for the peer-load kernels (push, staged); 0 = one per SM")
    ap.add_argument("--phases", action="store_true")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank, world, _ = init_dist()
    dtype = getattr(torch, a.dtype)
    es = torch.empty((), dtype=dtype).element_size()
    comm = make_comm(max(a.bytes))
    rows = []

    def emit(row):
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    from .._lib import lib
    for nbytes in a.bytes:
        comm.free_all()
        buf = comm.alloc(nbytes // es, dtype)
        fill(buf, rank)
        if comm.has_nvls:
            for th, un, wk, ln, sp, cps in itertools.product(a.threads, a.unroll, a.weak, a.lanes, a.stripe, a.ctas_per_sm):
                comm.set_nvls_config(threads=th, unroll=un, weak=wk, max_lanes=ln, stripe_bytes=sp)
                lib().ft_comm_set_nvls_ctas_per_sm(comm._h, cps)
                ms = time_collective(lambda: comm.all_reduce(buf, algo="nvls", op="avg"), a.iters, a.warmup)
                comm.check()
                emit({"bench": "nvls_sweep", "world": world, "bytes": nbytes, "dtype": a.dtype, "threads": th, "unroll": un, "weak": wk,
                      "max_lanes": ln, "stripe": sp, "ctas_per_sm": cps, "ms": round(ms, 5), "busbw_GBps": round(busbw(nbytes, ms, world), 1)})
            comm.set_nvls_config(threads=512, unroll=4, weak=0, max_lanes=0, stripe_bytes=0)
            lib().ft_comm_set_nvls_ctas_per_sm(comm._h, 1)
        for other in a.others:
            lane_caps = a.peer_lanes if other in ("push", "staged") else [0]
            for cap in lane_caps:
                if other == "nccl":
                    fn = lambda: dist.all_reduce(buf, op=dist.ReduceOp.AVG)  # noqa: E731
                elif other == "staged":
                    fn = lambda: comm.all_reduce(buf, algo="staged", op="avg")  # noqa: E731
                else:
                    if other == "hybrid" and not comm.has_nvls:
                        continue
                    fn = lambda other=other: comm.all_reduce(buf, algo=other, op="avg")  # noqa: E731
                comm.set_max_lanes(cap)     # 0: one CTA per SM
                ms = time_collective(fn, a.iters, a.warmup)
                comm.set_max_lanes(0)
                comm.check()
                emit({"bench": "nvls_sweep", "world": world, "bytes": nbytes, "dtype": a.dtype, "impl": other, "peer_lanes": cap,
                      "ms": round(ms, 5), "busbw_GBps": round(busbw(nbytes, ms, world), 1)})
        if a.phases:
            halves = {}
            for label, on in (("multimem", 2), ("peer loads", 0)):
                if on and not comm.has_nvls:
                    continue
                lib().ft_comm_set_phase_nvls(comm._h, on)
                halves[label] = (time_collective(lambda: comm.reduce_scatter(buf, op="avg"), a.iters, a.warmup),
                                 time_collective(lambda: comm.all_gather(buf), a.iters, a.warmup))
                comm.check()
            lib().ft_comm_set_phase_nvls(comm._h, 1)
            shard = torch.empty(nbytes // es // world, dtype=dtype, device=buf.device)
            loc = torch.empty(nbytes // es, dtype=dtype, device=buf.device)
            halves["nccl"] = (time_collective(lambda: dist.reduce_scatter_tensor(shard, loc, op=dist.ReduceOp.AVG), a.iters, a.warmup),
                              time_collective(lambda: dist.all_gather_into_tensor(loc, shard), a.iters, a.warmup))
            for label, (rs, ag) in halves.items():
                emit({"bench": "phases", "world": world, "bytes": nbytes, "dtype": a.dtype, "impl": label, "reduce_scatter_ms": round(rs, 5),
                      "all_gather_ms": round(ag, 5), "rs_busbw_GBps": round(busbw(nbytes, rs, world) / 2, 1),
                      "ag_busbw_GBps": round(busbw(nbytes, ag, world) / 2, 1)})
            del shard, loc
        del buf
    if rank == 0 and a.out:
        with open(a.out, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
