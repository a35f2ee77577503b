"""GPU-vs-CPU n-way reduce benchmark (single B200).

For each fan-in n the inputs are n vectors of ``--elems`` elements (uniform [-1,1), seeded);
each vector is larger than the 126 MB L2 at the default size, so every iteration streams
from HBM.  Reports effective bandwidth ``(n+1) * bytes / t`` from CUDA-event times and its
fraction of the measured copy bandwidth, and verifies the GPU result against the CPU kernel.
One JSON line per configuration.

Counterpart of the reference's vector_add benchmark (vector_add/vector_add.cu:49-203:
150 M floats, n = 1..16, 10 rounds, integer-millisecond host timer, no result recorded).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch

from ..ops import cpu_reduce, reduce_nway
from ..utils import cuda_time


def measured_hbm_gbs() -> tuple[float, str]:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def run(n: int, elems: int, dtype: torch.dtype, variant: int, iters: int, warmup: int, check: bool, cpu: bool, b2b: int = 0) -> dict:
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(1234 + n)
    ts = [(torch.rand(elems, generator=g, device=dev) * 2 - 1).to(dtype) for _ in range(n)]
    out = torch.empty_like(ts[0])
    if b2b > 0:   # `b2b` launches back to back between one pair of events (inputs larger than L2, no flush):
        ms = []   # what a training step or the headline benchmark sees, without the ramp of a lone launch
        for _ in range(warmup):
            reduce_nway(ts, out=out, variant=variant)
        for _ in range(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(b2b):
                reduce_nway(ts, out=out, variant=variant)
            e.record()
            e.synchronize()
            ms.append(s.elapsed_time(e) / b2b)
    else:
        ms = cuda_time(lambda: reduce_nway(ts, out=out, variant=variant), iters=iters, warmup=warmup, flush=True)
    t = statistics.median(ms)
    nbytes = elems * ts[0].element_size()
    gbs = (n + 1) * nbytes / (t * 1e-3) / 1e9
    peak, how = measured_hbm_gbs()
    row = {"bench": "reduce_nway", "n": n, "elems": elems, "dtype": str(dtype).split(".")[-1], "variant": variant, "back_to_back": b2b,
           "ms_median": round(t, 4), "ms_min": round(min(ms), 4), "GBps": round(gbs, 1),
           "frac_of_hbm": round(gbs / peak, 3), "hbm_peak_GBps": peak, "peak_source": f"of {how}"}
    if check or cpu:
        host = [x.cpu() for x in ts]
        t0 = time.perf_counter()
        want = cpu_reduce(host)
        cpu_s = time.perf_counter() - t0
        if cpu:
            row["cpu_ms"] = round(cpu_s * 1e3, 2)
            row["cpu_GBps"] = round((n + 1) * nbytes / cpu_s / 1e9, 1)
        tol = 1e-5 if dtype == torch.float32 else 4e-2
        err = (out.cpu().float() - want.float()).abs().max().item()
        row["max_abs_err_vs_cpu"] = err
        row["ok"] = err <= tol
    return row


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--fanin", type=int, nargs="+", default=[2, 3, 4, 8])
    ap.add_argument("--elems", type=int, default=64 << 20)
    ap.add_argument("--dtypes", nargs="+", default=["float32", "bfloat16"])
    ap.add_argument("--variants", type=int, nargs="+", default=[0])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true", help="verify against the CPU kernel")
    ap.add_argument("--cpu", action="store_true", help="also time the CPU kernel")
    ap.add_argument("--b2b", type=int, default=0, help="time this many launches back to back per sample instead of lone launches after an L2 flush")
    ap.add_argument("--out", default=None, help="append JSON lines to this file")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("this benchmark times the GPU kernels and needs a CUDA device; for the host reduction alone run "
              "allreduce_over_mpi_b200/lib/reduce_bench --cpu-only", file=sys.stderr)
        return 2
    rows = []
    for dt in a.dtypes:
        for n in a.fanin:
            for v in a.variants:
                row = run(n, a.elems, getattr(torch, dt), v, a.iters, a.warmup, a.check, a.cpu, a.b2b)
                rows.append(row)
                line = json.dumps(row)
                print(line, flush=True)
                if a.out:
                    with open(a.out, "a") as f:
                        f.write(line + "\n")
    return rows


if __name__ == "__main__":
    sys.exit(0 if main() is not None else 1)
