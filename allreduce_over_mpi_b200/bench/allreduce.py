"""All-reduce bus-bandwidth benchmark: FlexTree kernels vs NCCL on the same GPUs.

Launch one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        -m allreduce_over_mpi_b200.bench.allreduce --min-bytes 1024 --max-bytes 1073741824 \
        --dtypes float32 bfloat16 --shapes auto 8 2*4 4*2 2*2*2 --algos staged oneshot nvls --nccl

Every timing is a CUDA-event interval on the launching stream after warm-up; L2 is flushed
between timed iterations; the reported time is the median over iterations of the MAX over
ranks; busbw = bytes / t * 2(N-1)/N.  One JSON line per (size, dtype, implementation).

Counterpart of the reference's benchmark driver (allreduce_over_mpi/benchmark.cpp:31-243:
--size/--repeat/--comm-type/--check/--to-file, MPI_Wtime on rank 0, default 35 floats) with
NCCL in the place of the MPI library's own MPI_Allreduce as the comparison arm.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

from ..parallel.comm import FlexTreeComm
from ..parallel.planner import Shape, validate_shape
from ..utils import flush_l2


def init_dist() -> tuple[int, int, int]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, world, local


def time_collective(fn, iters: int, warmup: int, flush: bool = True) -> float:
    """Median over iterations of the max-over-ranks device time of ``fn`` in milliseconds."""
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        if flush:
            flush_l2()
        starts[i].record()
        fn()
        stops[i].record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) for a, b in zip(starts, stops)], dtype=torch.float64, device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return statistics.median(ms.tolist())


# Roofline of an all-reduce on NVSwitch: each GPU must take in 2(N-1)/N * S bytes over its links, so the
# bus bandwidth cannot exceed the per-direction link bandwidth; 770 GB/s is the measured peer-copy rate
# (calibration; 900 GB/s nominal).  The HBM side (at most ~3 S bytes per GPU) is an order of magnitude below its roof.
LINK_GBPS = 770.0


def busbw(nbytes: int, ms: float, world: int) -> float:
    return nbytes / (ms * 1e-3) / 1e9 * (2 * (world - 1) / world)


def fill(t: torch.Tensor, rank: int, it: int = 0):
    g = torch.Generator(device=t.device).manual_seed(1000 * it + rank)
    t.copy_((torch.rand(t.numel(), generator=g, device=t.device) * 2 - 1).to(t.dtype))


def expected(count: int, dtype, world: int, device, it: int = 0) -> torch.Tensor:
    acc = torch.zeros(count, dtype=torch.float64, device=device)
    tmp = torch.empty(count, dtype=dtype, device=device)
    for r in range(world):
        fill(tmp, r, it)
        acc += tmp.double()
    return acc


def sweep(a, comm: FlexTreeComm, rank: int, world: int) -> list[dict]:
    rows = []
    sizes = []
    s = a.min_bytes
    while s <= a.max_bytes:
        sizes.append(s)
        s *= a.step
    dev = comm.device
    if "all" in a.shapes:   # every executable shape for this world, cost model's pick first
        from ..parallel.planner import executable_shapes
        a.shapes = ["auto"] + [str(x) for x in executable_shapes(world)]
    for dt_name in a.dtypes:
        dtype = getattr(torch, dt_name)
        es = torch.empty((), dtype=dtype).element_size()
        for nbytes in sizes:
            count = nbytes // es
            comm.free_all()
            sym = comm.alloc(count, dtype)          # zero-copy path
            loc = torch.empty(count, dtype=dtype, device=dev)   # staged path / NCCL
            iters = a.iters if nbytes <= (64 << 20) else max(3, a.iters // 2)
            impls = []
            for shape in a.shapes:
                for algo in a.algos:
                    if algo == "none":     # only the comparison arm (--nccl)
                        continue
                    if algo == "lltree":   # the plan of every listed shape on tagged words (small messages)
                        if shape != "auto" and nbytes <= (64 << 10) and not validate_shape(world, Shape.parse(shape)):
                            impls.append((shape, algo))
                        continue
                    if algo != "staged" and shape != a.shapes[0]:
                        continue
                    if algo == "oneshot" and nbytes > min(comm.staging_bytes, a.oneshot_cap):
                        continue
                    if algo == "ll" and nbytes > (256 << 10):
                        continue
                    if algo in ("nvls", "hybrid") and (not comm.has_nvls or nbytes % 16):
                        continue
                    if algo == "nvls1" and (not comm.has_nvls or nbytes > min(comm.staging_bytes, a.nvls1_cap)):
                        continue
                    if algo == "hybrid":
                        if nbytes >= a.hybrid_min:
                            impls += [(f"{bf},{lf}", "hybrid") for bf, lf in a.hybrid]
                        continue
                    if algo == "staged" and shape != "auto" and validate_shape(world, Shape.parse(shape)):
                        continue
                    impls.append((shape, algo))
            for shape, algo in impls:
                label = f"flextree/{algo}/{shape}"
                if shape == "auto" and algo == "staged":
                    # "auto": whatever the cost model picks for this size
                    name, shp = comm.choose(nbytes, True, dtype)
                    fn = lambda: comm.all_reduce(sym)  # noqa: E731
                    label = f"flextree/auto->{name}/{shp}"
                elif algo == "staged":
                    fn = lambda shape=shape: comm.all_reduce(sym, shape=shape, algo="staged")  # noqa: E731
                elif algo == "nvls":
                    fn = lambda: comm.all_reduce(sym, algo="nvls")  # noqa: E731
                elif algo == "push":
                    fn = lambda: comm.all_reduce(sym, algo="push")  # noqa: E731
                elif algo == "hybrid":
                    bf, lf = (float(x) for x in shape.split(","))
                    comm.set_hybrid(bf, lf)
                    fn = lambda: comm.all_reduce(sym, algo="hybrid")  # noqa: E731
                    label = f"flextree/hybrid-{bf}-{lf}/{world}"
                elif algo == "nvls1":
                    fn = lambda: comm.all_reduce(loc, algo="nvls1")  # noqa: E731
                elif algo == "lltree":
                    fn = lambda shape=shape: comm.all_reduce(loc, shape=shape, algo="ll")  # noqa: E731
                elif algo == "ll":
                    fn = lambda: comm.all_reduce(loc, algo="ll")  # noqa: E731
                else:
                    fn = lambda: comm.all_reduce(loc, algo="oneshot")  # noqa: E731
                row = {"bench": "allreduce", "impl": label, "bytes": nbytes, "dtype": dt_name, "world": world}
                if a.check:
                    tgt = loc if algo in ("oneshot", "ll", "lltree", "nvls1") else sym
                    fill(tgt, rank)
                    fn()
                    torch.cuda.synchronize()
                    want = expected(count, dtype, world, dev)
                    err = (tgt.double() - want).abs().max().item()
                    row["max_abs_err"] = err
                    row["ok"] = err <= (1e-4 if dtype == torch.float32 else 0.25) * max(1.0, world / 8)
                    comm.check()
                ms = time_collective(fn, iters, a.warmup, flush=not a.no_flush)
                comm.check()
                row.update(ms=round(ms, 5), algbw_GBps=round(nbytes / ms / 1e6, 2), busbw_GBps=round(busbw(nbytes, ms, world), 2),
                           frac_of_link_roofline=round(busbw(nbytes, ms, world) / LINK_GBPS, 3))
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
            if a.staged_copy and nbytes <= comm.staging_bytes:
                fn = lambda: comm.all_reduce(loc, shape=Shape.flat(world), algo="staged")  # noqa: E731
                ms = time_collective(fn, iters, a.warmup, flush=not a.no_flush)
                row = {"bench": "allreduce", "impl": "flextree/staged-through-slots/flat", "bytes": nbytes, "dtype": dt_name,
                       "world": world, "ms": round(ms, 5), "busbw_GBps": round(busbw(nbytes, ms, world), 2)}
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
            if a.nccl:
                ms = time_collective(lambda: dist.all_reduce(loc), iters, a.warmup, flush=not a.no_flush)
                row = {"bench": "allreduce", "impl": "nccl", "bytes": nbytes, "dtype": dt_name, "world": world,
                       "ms": round(ms, 5), "algbw_GBps": round(nbytes / ms / 1e6, 2), "busbw_GBps": round(busbw(nbytes, ms, world), 2),
                       "frac_of_link_roofline": round(busbw(nbytes, ms, world) / LINK_GBPS, 3)}
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
            del sym, loc
    return rows


def make_comm(max_bytes: int, staging: int = 64 << 20, extra: int = 0) -> FlexTreeComm:
    return FlexTreeComm(heap_bytes=max_bytes + (4 << 20) + extra, staging_bytes=staging)


def phase_times(a, comm: FlexTreeComm, rank: int, world: int) -> list[dict]:
    """Device time of the two halves of the staged all-reduce, each issued as a call of its own (max over ranks)."""
    rows = []
    for dt_name in a.dtypes:
        dtype = getattr(torch, dt_name)
        es = torch.empty((), dtype=dtype).element_size()
        nbytes = a.min_bytes
        while nbytes <= a.max_bytes:
            for text in a.shapes:
                shape = None if text == "auto" else text
                comm.free_all()
                t = comm.alloc(max(1, nbytes // es), dtype)
                fill(t, rank)
                times = comm.profile_phases(t, shape=shape, iters=a.iters)
                v = torch.tensor([times["reduce_scatter_ms"], times["all_gather_ms"]], dtype=torch.float64, device="cuda")
                dist.all_reduce(v, op=dist.ReduceOp.MAX)
                comm.check()
                row = {"bench": "allreduce_phases", "bytes": nbytes, "dtype": dt_name, "world": world, "shape": times["shape"],
                       "reduce_scatter_ms": round(v[0].item(), 5), "all_gather_ms": round(v[1].item(), 5)}
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
            nbytes *= a.step
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--step", type=int, default=4)
    ap.add_argument("--dtypes", nargs="+", default=["float32"])
    ap.add_argument("--shapes", nargs="+", default=["auto"])
    ap.add_argument("--algos", nargs="+", default=["staged", "ll", "oneshot", "nvls"])
    ap.add_argument("--oneshot-cap", type=int, default=4 << 20)
    ap.add_argument("--nvls1-cap", type=int, default=16 << 20, help="largest message tried with the one-shot form through the switch")
    ap.add_argument("--hybrid", nargs="*", default=["0.7,0.5"], help="byte_fraction,lane_fraction pairs tried by algo hybrid")
    ap.add_argument("--hybrid-min", type=int, default=4 << 20)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--staged-copy", action="store_true", help="also time the path for tensors outside the symmetric heap")
    ap.add_argument("--out", default=None)
    ap.add_argument("--phases", action="store_true",
                    help="instead of the sweep: time the reduce-scatter and the all-gather half separately (staged, heap tensors)")
    a = ap.parse_args(argv)
    a.hybrid = [tuple(float(x) for x in h.split(",")) for h in a.hybrid]
    rank, world, _ = init_dist()
    comm = make_comm(a.max_bytes)
    if rank == 0:
        print(json.dumps({"bench": "allreduce", "world": world, "nvls": comm.has_nvls, "mem_kind": comm.mem_kind}), flush=True)
    rows = phase_times(a, comm, rank, world) if a.phases else sweep(a, comm, rank, world)
    if rank == 0 and a.out:
        with open(a.out, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    bad = [r for r in rows if r.get("ok") is False]
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    return 1 if bad else 0


# ---- entry used by the repository's bench.py ---------------------------------------------
def bench_allreduce_main(a) -> dict:
    """Headline number: in-place all-reduce of ``a.bytes`` in the symmetric heap, ``a.steps`` timed steps."""
    from ..ops import launch_count
    from ..utils import ClockSampler
    rank, world, local = init_dist()
    dtype = getattr(torch, a.dtype)
    es = torch.empty((), dtype=dtype).element_size()
    count = a.bytes // es
    chunk = getattr(a, "e2e_chunk", 16 << 20)
    comm = make_comm(a.bytes, extra=0 if a.no_e2e else 3 * chunk + (1 << 20))
    buf = comm.alloc(count, dtype)
    fill(buf, rank)
    comm.all_reduce(buf)
    torch.cuda.synchronize()
    err = (buf.double() - expected(count, dtype, world, comm.device)).abs().max().item()
    comm.check()
    name, shp = comm.choose(a.bytes, True, dtype)
    warm = max(a.warmup, 3)
    sampler = ClockSampler(gpu_index=local).start() if rank == 0 else None
    fill(buf, rank)

    # "avg" = sum with the 1/N factor fused into the reduction's store: the buffer is reduced in place step after
    # step and stays in [-1, 1) instead of growing by N per step
    def step():
        comm.all_reduce(buf, op="avg")

    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    l0 = launch_count()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.steps):
        step()
    e.record()
    torch.cuda.synchronize()
    launches = launch_count() - l0
    dist.barrier()
    t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / a.steps
    comm.check()
    finite = bool(torch.isfinite(buf).all().item())
    # keep the same load running (untimed) until the clock sampler has seen ~0.8 s of it
    for _ in range(min(4000, int(800.0 / max(ms, 1e-3)) + 1)):
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    nccl_ms = time_collective(lambda: dist.all_reduce(buf, op=dist.ReduceOp.AVG), min(a.steps, 10), warm, flush=False)
    per_gpu = busbw(a.bytes, ms, world)
    nccl_per_gpu = busbw(a.bytes, nccl_ms, world)
    res = {
        "metric": "all-reduce bus bandwidth GB/s per GPU; busbw = bytes/t * 2(N-1)/N, t = max over ranks",
        "value": round(per_gpu, 1), "per_gpu_busbw_GBps": round(per_gpu, 1), "whole_job_GBps": round(per_gpu * world, 1),
        "value_is": "bus bandwidth each GPU sustains (the conventional figure); all N GPUs sustain it at once, whole_job_GBps = N x value",
        "unit": "GB/s", "n_gpus": world, "steps": a.steps, "warmup": warm,
        "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": a.dtype, "data": "synthetic uniform[-1,1) seeded per rank",
        # `config` names the workload only and is spelled identically by the reference arm; what this arm does with it is in `details`
        "config": {"model": "all-reduce", "message_bytes": a.bytes, "global_batch": None, "seq_len": None,
                   "parallelism": f"dp{world}",
                   "l2": "input larger than L2" if a.bytes > (126 << 20) else "input smaller than L2, not flushed inside the back-to-back loop"},
        "details": {"algorithm": name, "shape": str(shp), "in_place": "symmetric heap (zero copy)",
                    "op": "avg (sum, 1/N fused into the store)"},
        "impl": "flextree", "nvls": comm.has_nvls, "max_abs_err_first_call": err, "finite_after_timed_steps": finite,
        "nccl_same_buffer": {"ms": round(nccl_ms, 5), "busbw_GBps": round(nccl_per_gpu, 1), "whole_job_GBps": round(nccl_per_gpu * world, 1)},
        "frac_of_nvlink_770GBps": round(per_gpu / 770.0, 3),
        "frac_of_nvls_roofline": round(per_gpu / (770.0 * 2 * (world - 1) / (world + 1)), 3),
        "scaling_note": "per-GPU message size is fixed (weak scaling); the 1-GPU run of this benchmark measures the n-way reduce kernel "
                        "(HBM-bound, no link involved), so its value is not comparable with the values at N > 1",
        "gpu_launches": int(launches), "clocks": clocks, "algorithms_used": comm.stats(),
    }
    if not a.no_e2e:
        res["e2e"] = e2e_allreduce(a, comm, buf, count, dtype, world)
    if not a.no_sweep:
        ns = argparse.Namespace(min_bytes=1024, max_bytes=min(a.bytes, 1 << 30), step=16, dtypes=[a.dtype], shapes=["auto"],
                                algos=["staged"], oneshot_cap=4 << 20, nvls1_cap=16 << 20, iters=10, warmup=3, nccl=True, check=False,
                                no_flush=False, staged_copy=False, hybrid=[], hybrid_min=1 << 62)
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):
            rows = sweep(ns, comm, rank, world)
        res["sweep"] = [{k: r[k] for k in ("impl", "bytes", "ms", "busbw_GBps")} for r in rows]
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    return res


def e2e_allreduce(a, comm, buf, count, dtype, world) -> dict:
    """The same message end to end through the public API for operands in host memory
    (``comm.all_reduce_host``, what ``MPI_Allreduce_FT`` runs for host buffers): every step takes the whole input
    from pinned host memory and leaves the WHOLE result in pinned host memory; both copies are inside the timed
    region and are pipelined chunk by chunk with the NVLink all-reduce."""
    # the pinned buffers go on the GPU's side of the host (first touch after moving this process next to the GPU)
    from ..utils.numa import bind_to_gpu_node
    placed = bind_to_gpu_node(comm.device.index) if os.environ.get("FT_NUMA_BIND", "1") != "0" else None
    g = torch.Generator().manual_seed(77 + comm.rank)
    host = torch.empty(count, dtype=dtype).pin_memory()
    host.copy_((torch.rand(count, generator=g) * 2 - 1).to(dtype))
    out = torch.empty(count, dtype=dtype).pin_memory()
    lib_chunk = getattr(a, "e2e_chunk", 16 << 20)
    from .._lib import lib
    lib().ft_comm_set_host_chunk(comm._h, lib_chunk)
    steps = max(2, min(a.steps, 5))

    def step():
        comm.all_reduce_host(host, out=out, op="avg")

    step()
    torch.cuda.synchronize()
    # check against the same sum made by NCCL from the same host data
    ref = host.to(comm.device).float()
    dist.all_reduce(ref)
    err = (out.to(comm.device).float() - ref / world).abs().max().item()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        step()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / steps
    comm.check()
    nbytes = count * host.element_size()
    per_gpu = busbw(nbytes, ms, world)
    return {"value": round(per_gpu, 1), "per_gpu_busbw_GBps": round(per_gpu, 1), "whole_job_GBps": round(per_gpu * world, 1),
            "unit": "GB/s", "ms_per_step": round(ms, 4), "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "steps": steps,
            "max_abs_err": err, "chunk_bytes": lib_chunk, "host_buffers_next_to_gpu": placed,
            "api": "FlexTreeComm.all_reduce_host (pinned host in, whole result to pinned host, chunked and overlapped)"}


if __name__ == "__main__":
    sys.exit(main())
