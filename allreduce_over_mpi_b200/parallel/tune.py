"""Calibration of the NVSwitch cost model from measured all-reduce sweeps.

    python -m allreduce_over_mpi_b200.parallel.tune sweep_8gpu.jsonl sweep_4gpu.jsonl ... \
        --out allreduce_over_mpi_b200/parallel/calibration_b200.json

Input: JSON lines written by ``bench/allreduce.py`` (one per size x implementation).
Output: a calibration file with
  * ``params``  - the v1 model's constants fitted by least squares: per-call launch cost,
    per-rendezvous latency, per-stage floor, achieved link bandwidth (best staged shape at
    the largest size), link efficiency as a function of how many peers a stage pulls from at
    once, one-shot limit and NVLS bandwidth;
  * ``table``   - per world size, the measured winner (algorithm, shape) per message size,
    which the communicator consults before falling back to the model;
  * ``fit``     - predicted vs measured time per row, so the model's error is on record
    (``python -m allreduce_over_mpi_b200.parallel.tune --report [calibration.json]`` prints a summary).

This is the re-derivation, on measured B200 numbers, of the reference's constants lo / co /
bo / o (cost_model/CostModel.h:3-4, :24, :37), which were fitted to a 16-host Ethernet cluster.
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import defaultdict

from . import planner
from .planner import CostParams, Shape


def parse_rows(paths):
    rows = []
    for p in paths:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{") and '"impl"' in line:
                    rows.append(json.loads(line))
    return rows


def split_impl(impl: str):
    """'flextree/staged/2*4' -> ('staged', '2*4'); 'flextree/auto->nvls/8' -> None (derived rows are skipped)."""
    parts = impl.split("/")
    if parts[0] != "flextree" or "auto->" in impl or len(parts) < 3:
        return None
    if parts[1].startswith("hybrid-"):
        return parts[1], parts[2]   # 'hybrid-<byte fraction>-<lane fraction>'
    if parts[1] not in ("staged", "oneshot", "nvls", "nvls1", "ll", "lltree", "push"):
        return None
    return parts[1], parts[2]   # 'lltree' = a plan on tagged words: becomes an "ll" row that keeps its shape


def best_table(rows) -> dict:
    by = defaultdict(lambda: defaultdict(list))
    for r in rows:
        k = split_impl(r["impl"])
        if k is None or r.get("ok") is False:
            continue
        algo, shape = k
        if algo == "lltree":
            algo = "ll"
        elif algo != "staged":
            shape = str(r["world"])
        elif shape == "auto":
            continue
        by[r["world"]][r["bytes"]].append((r["ms"], algo, shape))
    table = {}
    for world, sizes in by.items():
        out = []
        for nbytes in sorted(sizes):
            ms, algo, shape = min(sizes[nbytes])
            out.append([nbytes, algo, shape, round(ms * 1e3, 2)])
        table[str(world)] = out
    return table


def fit_params(rows) -> tuple[CostParams, list]:
    """Least-squares fit of the v1 constants to the staged rows; closed forms for the rest."""
    p = CostParams()
    staged = []
    for r in rows:
        k = split_impl(r["impl"])
        if k and k[0] == "staged" and k[1] != "auto" and r.get("ok") is not False:
            staged.append((r["world"], Shape.parse(k[1]), r["bytes"], r["ms"] * 1e3))
    if not staged:
        return p, []
    # latency terms from the smallest size: t = launch + sync * (stages + 1)
    small = min(b for _, _, b, _ in staged)
    pts = [(planner.plan_num_stages(w, s), us) for w, s, b, us in staged if b == small]
    n = len(pts)
    p.stage_floor_us = 0.0
    if n >= 2:
        sx = sum(x for x, _ in pts); sy = sum(y for _, y in pts)
        sxx = sum(x * x for x, _ in pts); sxy = sum(x * y for x, y in pts)
        den = n * sxx - sx * sx
        slope = (n * sxy - sx * sy) / den if den else 0.0
        icpt = (sy - slope * sx) / n
        p.sync_us = max(0.1, slope)
        p.launch_us = max(0.0, icpt - p.sync_us)

    def wire_us(w, s, us):   # what is left of a measurement once the fixed costs are taken out
        return max(us - p.launch_us - p.sync_us * (planner.plan_num_stages(w, s) + 1), 1e-3)

    # link bandwidth: the best staged shape at the largest size moves 2(N-1)/N * S per direction
    big = max(b for _, _, b, _ in staged)
    p.link_gbs = max(2 * (w - 1) / w * b / (wire_us(w, s, us) * 1e-6) / 1e9 for w, s, b, us in staged if b == big)
    # peer efficiency: for every fan-out k (peers pulled at once), ratio of the bandwidth a shape
    # whose widest stage has k peers reaches at the largest size to the best one
    eff = defaultdict(float)
    for w, s, b, us in staged:
        if b != big or s.ring or s.lonely:
            continue
        k = max(s.widths) - 1
        bw = 2 * (w - 1) / w * b / (wire_us(w, s, us) * 1e-6) / 1e9
        eff[k] = max(eff[k], min(1.0, bw / p.link_gbs))
    p.peer_eff = {int(k): round(v, 3) for k, v in eff.items()}
    # NVLS: bytes through each GPU's links are S * (1 + 1/N)
    nv = [(r["world"], r["bytes"], r["ms"] * 1e3) for r in rows if (split_impl(r["impl"]) or ("", ""))[0] == "nvls"]
    if nv:
        w, b, us = max(nv, key=lambda t: t[1])
        p.nvls_gbs = b * (1 + 1 / w) / (max(us - p.launch_us - 3 * p.sync_us, 1e-3) * 1e-6) / 1e9
    # low-latency protocol: its fixed cost is the fastest time at the smallest size
    ll = [r["ms"] * 1e3 for r in rows if (split_impl(r["impl"]) or ("", ""))[0] == "ll" and r["bytes"] <= 4096]
    if ll:
        p.ll_us = min(ll)
    # reduce+push: how much faster its write half runs than the read half, from the largest size
    pu = [(r["world"], r["bytes"], r["ms"] * 1e3) for r in rows if (split_impl(r["impl"]) or ("", ""))[0] == "push"]
    if pu:
        w, b, us = max(pu, key=lambda t: t[1])
        half = b * (w - 1) / w
        eff = p.peer_eff.get(w - 1, 1.0)
        t_read = half / (p.link_gbs * eff) * 1e-3
        t_write = max(us - p.launch_us - 2 * p.sync_us - t_read, 1e-3)
        p.push_gain = round(max(0.5, min(2.0, t_read / t_write)), 3)
    # one-shot limit: largest size at which one-shot still beats every staged shape
    os_rows = defaultdict(dict)
    for r in rows:
        k = split_impl(r["impl"])
        if k:
            os_rows[(r["world"], r["bytes"])].setdefault(k[0], []).append(r["ms"])
    lim = 0
    for (w, b), d in os_rows.items():
        if "oneshot" in d and "staged" in d and min(d["oneshot"]) <= min(d["staged"]):
            lim = max(lim, b)
    if lim:
        p.oneshot_max_bytes = float(lim)
    fit = []
    for w, s, b, us in staged:
        pred = planner.cost_v1(w, s, b, p)
        fit.append({"world": w, "shape": str(s), "bytes": b, "measured_us": round(us, 2), "predicted_us": round(pred, 2),
                    "rel_err": round((pred - us) / us, 3)})
    return p, fit


def report(path: str) -> str:
    """Predicted against measured, from the ``fit`` section of a calibration file: per world size the
    median and worst relative error of the model over the staged shapes, and how often the shape the
    model ranks first is the one that measured fastest (or within 3 % of it)."""
    with open(path) as f:
        doc = json.load(f)
    detail = doc.get("fit", {}).get("detail", [])
    out = [f"cost model v1 fit: {len(detail)} measured staged runs, median |error| {doc.get('fit', {}).get('median_abs_rel_err')}",
           "", "| world | runs | median abs err | worst err | sizes | model's first choice fastest (within 3 %) |", "|---|---|---|---|---|---|"]
    by_world = defaultdict(list)
    for d in detail:
        by_world[d["world"]].append(d)
    for world in sorted(by_world):
        rows = by_world[world]
        errs = sorted(abs(d["rel_err"]) for d in rows)
        worst = max(rows, key=lambda d: abs(d["rel_err"]))
        by_size = defaultdict(dict)
        for d in rows:   # a shape measured twice: keep the faster run
            t = by_size[d["bytes"]].get(d["shape"])
            if t is None or d["measured_us"] < t[0]:
                by_size[d["bytes"]][d["shape"]] = (d["measured_us"], d["predicted_us"])
        sizes = [b for b, shapes in by_size.items() if len(shapes) > 1]
        right = 0
        for b in sizes:
            shapes = by_size[b]
            pick = min(shapes, key=lambda k: shapes[k][1])
            best = min(v[0] for v in shapes.values())
            right += shapes[pick][0] <= best * 1.03
        out.append(f"| {world} | {len(rows)} | {errs[len(errs) // 2]:.3f} | {worst['rel_err']:+.3f} ({worst['shape']}, {worst['bytes']} B) | "
                   f"{len(sizes)} | {right} of {len(sizes)} |" if sizes else
                   f"| {world} | {len(rows)} | {errs[len(errs) // 2]:.3f} | {worst['rel_err']:+.3f} ({worst['shape']}, {worst['bytes']} B) | 0 | one shape only |")
    p = doc.get("params", {})
    out += ["", "fitted constants: " + ", ".join(f"{k} = {p[k]:.4g}" for k in ("launch_us", "sync_us", "stage_floor_us", "link_gbs", "nvls_gbs",
                                                                              "ll_us", "push_gain", "hbm_gbs") if k in p),
            "link efficiency by number of peers read at once: " + ", ".join(f"{k}: {v}" for k, v in sorted(p.get("peer_eff", {}).items(), key=lambda kv: int(kv[0])))]
    return "\n".join(out)


def main(argv=None):
    argv = sys.argv[1:] if argv is None else list(argv)
    if argv and argv[0] == "--report":
        print(report(argv[1] if len(argv) > 1 else planner.calibration_path()))
        return 0
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("sweeps", nargs="+")
    ap.add_argument("--out", default=planner.calibration_path())
    ap.add_argument("--dtype", default=None, help="only rows of this dtype (default: all)")
    ap.add_argument("--hbm-gbs", type=float, default=None, help="measured local copy bandwidth (read+write GB/s) for the model's HBM term")
    a = ap.parse_args(argv)
    rows = parse_rows(a.sweeps)
    if a.dtype:
        rows = [r for r in rows if r.get("dtype") == a.dtype]
    params, fit = fit_params(rows)
    if a.hbm_gbs:
        params.hbm_gbs = a.hbm_gbs
    table = best_table(rows)
    errs = [abs(f["rel_err"]) for f in fit]
    doc = {"params": json.loads(params.to_json()), "table": table,
           "fit": {"rows": len(fit), "median_abs_rel_err": round(sorted(errs)[len(errs) // 2], 3) if errs else None, "detail": fit},
           "source": a.sweeps}
    with open(a.out, "w") as f:
        json.dump(doc, f, indent=1)
    print(json.dumps({"out": a.out, "params": doc["params"], "median_abs_rel_err": doc["fit"]["median_abs_rel_err"],
                      "worlds": sorted(table)}, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
