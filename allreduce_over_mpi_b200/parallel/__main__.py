"""Command line of the planner and cost model: ``python -m allreduce_over_mpi_b200.parallel <command> ...``
(see :func:`main`).  Host only; no GPU is touched."""
from __future__ import annotations

import sys

from .planner import (CostParams, candidate_shapes, choose_v0, choose_width, count_ordered_factorizations, describe,
                      executable_shapes, parse_topo, pick_algorithm, rs_holders)

def main(argv=None) -> int:
    """``python -m allreduce_over_mpi_b200.parallel <command> ...`` - the reference's small tools in one place:

      factor-count N [N ...]        number of ordered factorisations (topo_count/factor_count.py)
      candidates N                  candidate tree shapes incl. the 1*N / N*1 sentinels (cost_model/GetWidth.h)
      choose-width N                shapes for N, and the +1 / -1 neighbours when N is prime (cost_model/ChooseWidth.h)
      choose N [chunk]              the v0 model's pick and cost (cost_model/CostModel.h)
      pick N BYTES                  the calibrated NVSwitch model's pick (algorithm, shape, predicted microseconds)
      shapes N                      every executable shape for N ranks
      describe N TOPO [LONELY]      every rank's schedule for FT_TOPO-style widths, e.g. ``describe 5 2,2 1``
      owners N TOPO [LONELY]        which rank holds which block after the reduce-scatter half
    """
    import argparse
    ap = argparse.ArgumentParser(prog="planner", description=main.__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["factor-count", "candidates", "choose-width", "choose", "pick", "shapes", "describe", "owners"])
    ap.add_argument("args", nargs="*")
    a = ap.parse_args(argv)
    try:
        if a.command == "factor-count":
            for n in a.args:
                print(count_ordered_factorizations(int(n)))
        elif a.command == "candidates":
            print("\n".join(candidate_shapes(int(a.args[0]))))
        elif a.command == "choose-width":
            print("\n".join(choose_width(int(a.args[0]))))
        elif a.command == "choose":
            shape, cost, ncand = choose_v0(int(a.args[0]), float(a.args[1]) if len(a.args) > 1 else 100.0)
            print(f"{shape} {cost:.6g} ({ncand} candidates)")
        elif a.command == "pick":
            algo, shape, us = pick_algorithm(int(a.args[0]), int(a.args[1]), CostParams.load())   # calibrated constants
            print(f"{algo} {shape} {us:.2f} us")
        elif a.command == "shapes":
            print("\n".join(str(s) for s in executable_shapes(int(a.args[0]))))
        else:
            world = int(a.args[0])
            shape, _ = parse_topo(a.args[1] if len(a.args) > 1 else None, a.args[2] if len(a.args) > 2 else None, world)
            if a.command == "describe":
                for r in range(world):
                    print(describe(world, shape, r), end="")
            else:
                for b, ranks in enumerate(rs_holders(world, shape)):
                    print(f"block {b}: rank {', '.join(map(str, ranks))}")
    except (IndexError, ValueError) as e:
        print(f"planner {a.command}: bad arguments ({e})", file=sys.stderr)
        return 2
    except Exception as e:  # noqa: BLE001 - invalid layouts come back as a message, as from the library
        print(str(e), file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
