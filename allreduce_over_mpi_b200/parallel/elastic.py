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


class RankLost(RuntimeError):
    """Raised on the host, between steps, when peers stopped reporting."""

    def __init__(self, lost):
        self.lost = set(lost)
        super().__init__(f"ranks {sorted(self.lost)} stopped reporting")


class Liveness:
    """Host-side liveness over a ``torch.distributed`` store (TCPStore, FileStore, HashStore).

    Every rank calls :meth:`beat` once per step (it bumps a counter under its own key) and
    :meth:`guard` before it launches the next collective.  A peer whose counter has not moved for
    ``timeout_s`` of this rank's own clock is reported lost, so the survivors learn of it on the
    host and never launch a kernel that would wait for it (the device-side wait limit remains the
    second line of defence).  No clocks are compared between ranks.  The store should live in a
    process that outlasts the ranks (the launcher's), or on a rank that is not expected to leave.
    """

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "ft/alive/"):
        import time
        self._now = time.monotonic
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self._count = 0
        t = self._now()
        self._seen = {r: (None, t) for r in range(world) if r != rank}
        self.beat()

    def beat(self):
        self._count += 1
        self.store.set(f"{self.prefix}{self.rank}", str(self._count))

    def leave(self):
        """Announce that this rank takes part in ONE more step and then stops.  Call it right before the
        :meth:`guard` of that last step.  The note carries the number of that step (ranks call :meth:`guard` once per
        step, so their counters agree): a peer that reads it while still on the same step carries on and launches; a
        peer on the step after it can only have got there by finishing a collective this rank took part in, which this
        rank launched after writing the note - so that peer is certain to see it before its next launch.  No peer ever
        launches a kernel that waits for a rank that has left, and nobody has to wait for a silence to time out."""
        self.store.set(f"{self.prefix}gone/{self.rank}", str(self._count + 1))

    def poll(self) -> set[int]:
        """Ranks that announced their departure, or have been silent for longer than the timeout."""
        now, lost = self._now(), set()
        for r, (last, since) in self._seen.items():
            gone = f"{self.prefix}gone/{r}"
            if self.store.check([gone]):
                if self._count > int(bytes(self.store.get(gone))):   # its last step is behind this rank
                    lost.add(r)
                continue
            key = f"{self.prefix}{r}"
            val = bytes(self.store.get(key)) if self.store.check([key]) else None
            if val != last:
                self._seen[r] = (val, now)
            elif now - since > self.timeout_s:
                lost.add(r)
        return lost

    def guard(self):
        """Call between steps: beat, then raise :class:`RankLost` if a peer has gone silent."""
        self.beat()
        lost = self.poll()
        if lost:
            raise RankLost(lost)
