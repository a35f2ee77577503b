#!/usr/bin/env python
"""Headline benchmark.

  python bench.py --gpus 1 --steps K --warmup W
      n-way reduce-sum on one B200: a step is one fp32 reduce for each fan-in n in {2,3,4,8}
      over 64 Mi-element vectors (inputs larger than L2); value = sum((n+1)*bytes) / time, GB/s.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
      FlexTree all-reduce over NVLink peer memory on N B200s: a step is one in-place all-reduce of
      --bytes (default 256 MiB) fp32 per GPU; per-GPU bus bandwidth = (bytes/t) * 2(N-1)/N in GB/s,
      t = max over ranks of CUDA-event time; value = N x that (the whole job), the per-GPU figure
      and the NCCL number for the same buffer ride along.

  --impl reference runs the unmodified reference code for the same metric (its CUDA reduce_sum_gpu
  launcher at N = 1, its MPI_Allreduce_FT over a shared-memory MPI shim at N > 1).

Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="flextree", choices=["flextree", "reference"])
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--elems", type=int, default=64 << 20, help="vector length of the 1-GPU n-way reduce")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-chunk", type=int, default=16 << 20, help="chunk size of the host pipelines in the end-to-end step")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


# ------------------------------------------------------------------------------ N = 1
FANINS = (2, 3, 4, 8)


def bench_nway(a) -> dict:
    import torch
    from allreduce_over_mpi_b200.ops import launch_count, reduce_nway
    from allreduce_over_mpi_b200.utils import ClockSampler

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    dtype = getattr(torch, a.dtype)
    elems = a.elems
    g = torch.Generator(device=dev).manual_seed(2024)
    vecs = [(torch.rand(elems, generator=g, device=dev) * 2 - 1).to(dtype) for _ in range(max(FANINS))]
    outs = {n: torch.empty_like(vecs[0]) for n in FANINS}
    nbytes = elems * vecs[0].element_size()
    step_bytes = sum((n + 1) * nbytes for n in FANINS)

    def step():
        for n in FANINS:
            reduce_nway(vecs[:n], out=outs[n])

    sampler = ClockSampler(gpu_index=0).start()   # runs through warm-up, the timed steps and a tail of the same load
    t_wall = time.time()
    for _ in range(max(a.warmup, 3)):
        step()
    torch.cuda.synchronize()
    per_n = {}
    l0 = launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(a.steps + 1)]
    torch.cuda.synchronize()
    ev[0].record()
    for i in range(a.steps):
        step()
        ev[i + 1].record()
    torch.cuda.synchronize()
    launches = launch_count() - l0
    while time.time() - t_wall < 1.0:   # same load, untimed, until the 100 ms clock sampler has seen enough of it
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    total_ms = ev[0].elapsed_time(ev[-1])
    ms_per_step = total_ms / a.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # per fan-in detail (same buffers, event pair around ONE launch).  A launch of the same kernel is queued just
    # before the pair, so the timed launch is already waiting in the stream when its turn comes and the interval holds
    # the kernel alone, not the host's time to issue it (tens of microseconds from Python, a tenth of these kernels).
    for n in FANINS:
        ms = []
        for _ in range(5):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reduce_nway(vecs[:n], out=outs[n])
            s.record(); reduce_nway(vecs[:n], out=outs[n]); e.record(); e.synchronize()
            ms.append(s.elapsed_time(e))
        t = statistics.median(ms)
        per_n[str(n)] = {"ms": round(t, 4), "GBps": round((n + 1) * nbytes / (t * 1e-3) / 1e9, 1)}
    # correctness of what was timed
    want = torch.stack([v.float() for v in vecs[:4]]).sum(0)
    err = (outs[4].float() - want).abs().max().item()
    del want
    # the same four fan-ins on bf16 vectors of the same length (fp32 accumulation, one rounding), untimed above
    per_n16 = {}
    if a.dtype == "float32":
        v16 = [v.to(torch.bfloat16) for v in vecs]
        o16 = torch.empty_like(v16[0])
        for n in FANINS:
            for _ in range(3):
                reduce_nway(v16[:n], out=o16)
            ms = []
            for _ in range(5):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reduce_nway(v16[:n], out=o16)
                s.record(); reduce_nway(v16[:n], out=o16); e.record(); e.synchronize()
                ms.append(s.elapsed_time(e))
            t = statistics.median(ms)
            per_n16[str(n)] = {"ms": round(t, 4), "GBps": round((n + 1) * nbytes / 2 / (t * 1e-3) / 1e9, 1)}
        want16 = torch.stack([v.float() for v in v16[:8]]).sum(0)
        per_n16["max_abs_err_n8"] = (o16.float() - want16).abs().max().item()
        del v16, o16, want16

    pk, how = peaks()
    res = {
        "metric": "n-way reduce-sum GB/s (sum over n in {2,3,4,8} of (n+1)*bytes / time)",
        "value": round(value, 1), "unit": "GB/s", "n_gpus": 1, "steps": a.steps, "warmup": max(a.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": a.dtype, "data": "synthetic uniform[-1,1) seeded",
        # `config` names the workload only and is spelled identically by the reference arm; what this arm does with it is in `details`
        "config": {"model": "n-way reduce-sum, n in {2,3,4,8}", "elems_per_vector": elems, "global_batch": None,
                   "seq_len": None, "parallelism": "single GPU", "l2": "inputs larger than L2"},
        "details": {"accumulate": "fp32", "kernel": "reduce_nway_wide_kernel (256-bit loads and stores)",
                    "bytes_per_vector": nbytes},
        "impl": "flextree", "per_fanin": per_n, "per_fanin_bf16": per_n16, "frac_of_hbm_copy_peak": round(value / pk["hbm_gbs"], 3),
        "peak_source": f"of {how} ({pk['hbm_gbs']} GB/s copy)", "max_abs_err": err,
        "gpu_launches": int(launches), "clocks": clocks,
        "scaling_note": "one GPU has no link to measure: this run times the n-way reduce kernel (HBM-bound), the runs at "
                        "N > 1 time the all-reduce (NVLink-bound); the two values are different quantities",
    }
    if not a.no_e2e:
        del outs
        res["e2e"] = e2e_nway(a, vecs, step_bytes)
    return res


def e2e_nway(a, vecs, step_bytes) -> dict:
    """The same step end to end through the public API for operands in host memory
    (``ops.HostReducePipeline``): every step copies the 8 input vectors from pinned host memory to the
    device, reduces the four fan-ins and copies the four results back to pinned host memory.  The copies are
    part of the timed region; the pipeline overlaps them chunk by chunk with each other and with the kernels."""
    import torch
    from allreduce_over_mpi_b200.ops import HostReducePipeline
    host_in = [torch.empty(v.shape, dtype=v.dtype).pin_memory() for v in vecs]
    for h, v in zip(host_in, vecs):
        h.copy_(v)
    host_out = [torch.empty(vecs[0].shape, dtype=vecs[0].dtype).pin_memory() for _ in FANINS]
    steps = max(2, min(a.steps, 4))
    pipe = HostReducePipeline(chunk_bytes=a.e2e_chunk, max_inputs=len(host_in), max_outputs=len(FANINS))

    def step():
        pipe.run(host_in, FANINS, host_out)

    step()
    torch.cuda.synchronize()
    want = torch.stack([h[:4096].float() for h in host_in[:FANINS[-1]]]).sum(0)
    err = (host_out[-1][:4096].float() - want).abs().max().item()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        step()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / steps
    pipe.close()
    h2d = sum(h.numel() * h.element_size() for h in host_in)
    d2h = sum(h.numel() * h.element_size() for h in host_out)
    return {"value": round(step_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(ms, 3),
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps, "max_abs_err": err,
            "api": "ops.HostReducePipeline.run (pinned host in, pinned host out, chunked and overlapped)",
            "chunk_bytes": a.e2e_chunk}


# ------------------------------------------------------------------------------ main
def main():
    a = parse()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    # Libraries (NCCL's version banner, torch warnings) may write to stdout; the contract is ONE JSON
    # line there.  Everything else goes to stderr until the result is ready.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        out = run(a, world, rank)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    if rank == 0 and out is not None:
        print(json.dumps(out), flush=True)
    return 0


def run(a, world, rank):
    if a.impl == "reference":
        from baseline.reference_arm import run_reference
        return run_reference(a, world, rank)
    if a.gpus <= 1 and world <= 1:
        return bench_nway(a)
    from allreduce_over_mpi_b200.bench.allreduce import bench_allreduce_main
    return bench_allreduce_main(a)


if __name__ == "__main__":
    sys.exit(main())
