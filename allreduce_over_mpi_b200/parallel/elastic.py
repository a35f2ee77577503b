"""Re-planning after a rank is lost (host-side; the reference has no elasticity at all).

A device-side wait that runs out reports which peer never arrived (`FlexTreeComm.check()`).  The
survivors can then form a smaller world; the lonely layouts of FlexTree exist precisely for
world sizes that do not factor, so the cost model is asked for the best executable shape of the
shrunken world.  Creating the new communicator (new process group, new symmetric heaps) is the
caller's job: memory bound to a multicast object must be released by every survivor first.
"""
from __future__ import annotations

from dataclasses import dataclass

from . import planner
from .planner import CostParams, Shape


@dataclass
class Replan:
    world: int                 # size of the surviving world
    rank_map: dict[int, int]   # old rank -> new rank (survivors only, order preserved)
    algo: str
    shape: Shape
    predicted_us: float
    candidates: list[str]      # every executable shape of the new world


def replan_after_failure(world: int, failed: set[int] | list[int], nbytes: int, params: CostParams | None = None,
                         nvls: bool = False) -> Replan:
    failed = set(failed)
    if not failed <= set(range(world)):
        raise ValueError("failed ranks outside the world")
    survivors = [r for r in range(world) if r not in failed]
    if not survivors:
        raise ValueError("no rank survives")
    n = len(survivors)
    algo, shape, us = planner.pick_algorithm(n, nbytes, params or CostParams.load(), allow_oneshot=True, allow_nvls=nvls)
    return Replan(n, {old: new for new, old in enumerate(survivors)}, algo, shape, us,
                  [str(s) for s in planner.executable_shapes(n)])
