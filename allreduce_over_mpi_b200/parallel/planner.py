"""Python face of the C++ planner, cost models and CPU executors.

Everything here calls into ``libflextree.so`` (``csrc/planner/*.hpp`` behind
``csrc/api/flextree_host.cpp``); nothing is re-implemented in Python.  Reference
counterparts: cost_model/*.h, topo_count/factor_count.py and the planner classes of
allreduce_over_mpi/mpi_mod.hpp:80-766 (also shipped as tmp_tree.cpp).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import threading
from dataclasses import dataclass, field
from typing import Sequence

import torch

from .._lib import FlexTreeError, V1Params, check, lib, text_call
from ..ops.reduce import ft_dtype
from .._lib import OPS


@dataclass(frozen=True)
class Shape:
    """Tree shape: bottom-up level widths, lonely ranks, or the ring."""
    widths: tuple[int, ...]
    lonely: int = 0
    ring: bool = False

    @staticmethod
    def parse(text: str) -> "Shape":
        """``"2*4"``, ``"2x2+1"``, ``"8"``, ``"ring8"``."""
        t = text.strip().lower()
        if t.startswith("ring"):
            return Shape((int(t[4:]),), 0, True)
        lonely = 0
        if "+" in t:
            t, l = t.split("+")
            lonely = int(l)
        widths = tuple(int(x) for x in t.replace("x", "*").replace(",", "*").split("*") if x)
        return Shape(widths, lonely, False)

    @staticmethod
    def flat(world: int) -> "Shape":
        return Shape((world,))

    @property
    def world(self) -> int:
        if self.ring:
            return self.widths[0]
        n = 1
        for w in self.widths:
            n *= w
        return n + self.lonely

    def __str__(self) -> str:
        if self.ring:
            return f"ring{self.widths[0]}"
        return "*".join(map(str, self.widths)) + (f"+{self.lonely}" if self.lonely else "")

    def c_args(self):
        arr = (C.c_int * max(1, len(self.widths)))(*self.widths)
        return arr, len(self.widths), self.lonely, int(self.ring)


def _lines(s: str) -> list[str]:
    return [x for x in s.split("\n") if x]


# ---- factorisation tools ----------------------------------------------------------------
def prime_factors(n: int) -> list[int]:
    out = (C.c_int * 64)()
    k = lib().ft_prime_factors(n, out, 64)
    return list(out[:k])


def is_prime(n: int, loose: bool = False) -> bool:
    """``loose=True`` is the reference's predicate, which calls 1 prime."""
    return bool(lib().ft_is_prime_loose(n) if loose else lib().ft_is_prime(n))


def count_ordered_factorizations(n: int) -> int:
    return int(lib().ft_count_ordered_factorizations(n))


def candidate_shapes(n: int, legacy: bool = False) -> list[str]:
    """Candidate tree shapes for n ranks as ``"w0*w1*..."`` strings (incl. ``1*n`` / ``n*1``)."""
    return _lines(text_call(lib().ft_candidate_shapes, n, int(legacy)))


def choose_width(world: int) -> list[str]:
    """Shapes of ``world`` plus the ``-1`` / ``+1`` neighbours (lonely candidates)."""
    return _lines(text_call(lib().ft_choose_width, world))


def executable_shapes(world: int) -> list[Shape]:
    return [Shape.parse(s) for s in _lines(text_call(lib().ft_executable_shapes, world))]


# ---- cost models ------------------------------------------------------------------------
def cost_v0(widths: Sequence[int], n: int, chunk: float = 100.0) -> float:
    arr = (C.c_int * len(widths))(*widths)
    return float(lib().ft_cost_v0(arr, len(widths), n, chunk))


def choose_v0(n: int, chunk: float = 100.0) -> tuple[str, float, int]:
    """Arg-min of the original analytic model: (shape string, cost, candidates scored)."""
    w = (C.c_int * 64)()
    cost = C.c_double()
    ncand = C.c_uint64()
    k = lib().ft_choose_v0(n, chunk, w, 64, C.byref(cost), C.byref(ncand))
    return "*".join(str(w[i]) for i in range(k)), cost.value, int(ncand.value)


@dataclass
class CostParams:
    """Measured parameters of the NVSwitch cost model (v1); see csrc/planner/cost_model.hpp."""
    launch_us: float = 4.0
    sync_us: float = 2.5
    link_gbs: float = 700.0
    hbm_gbs: float = 6000.0
    stage_floor_us: float = 0.5
    nvls_gbs: float = 0.0
    oneshot_max_bytes: float = float(1 << 20)
    ll_us: float = 0.0            # fixed cost of the low-latency push protocol (0: not available)
    ll_max_bytes: float = float(256 << 10)
    push_gain: float = 0.0        # > 0: reduce+push kernel available; efficiency of posted writes relative to reads
    peer_eff: dict[int, float] = field(default_factory=dict)

    def to_c(self) -> V1Params:
        p = V1Params()
        lib().ft_v1_defaults(C.byref(p))
        for k in ("launch_us", "sync_us", "link_gbs", "hbm_gbs", "stage_floor_us", "nvls_gbs", "oneshot_max_bytes", "ll_us",
                  "ll_max_bytes", "push_gain"):
            setattr(p, k, float(getattr(self, k)))
        for k, v in self.peer_eff.items():
            p.peer_eff[int(k)] = float(v)
        return p

    def to_json(self) -> str:
        return json.dumps(self.__dict__, indent=1, sort_keys=True)

    @staticmethod
    def from_json(text: str) -> "CostParams":
        d = json.loads(text)
        d = d.get("params", d)   # a calibration file nests the parameters next to the choice table
        d = {k: v for k, v in d.items() if k in CostParams.__dataclass_fields__}
        d["peer_eff"] = {int(k): float(v) for k, v in d.get("peer_eff", {}).items()}
        return CostParams(**d)

    @staticmethod
    def load(path: str | os.PathLike | None = None) -> "CostParams":
        """Calibration table: ``path``, else $FT_CALIBRATION, else the packaged default."""
        path = path or os.environ.get("FT_CALIBRATION") or os.path.join(os.path.dirname(__file__), "calibration_b200.json")
        if os.path.exists(path):
            with open(path) as f:
                return CostParams.from_json(f.read())
        return CostParams()


def calibration_path(path: str | os.PathLike | None = None) -> str:
    return str(path or os.environ.get("FT_CALIBRATION") or os.path.join(os.path.dirname(__file__), "calibration_b200.json"))


def load_choice_table(path: str | os.PathLike | None = None) -> dict:
    """Measured winners per world size: {"8": [[bytes, algo, shape], ...]} (empty when not calibrated)."""
    path = calibration_path(path)
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("table", {})
    return {}


def cost_v1(world: int, shape: Shape, nbytes: int, params: CostParams | None = None) -> float:
    p = (params or CostParams()).to_c()
    return float(lib().ft_cost_v1(world, *shape.c_args(), nbytes, C.byref(p)))


def cost_v1_oneshot(world: int, nbytes: int, params: CostParams | None = None) -> float:
    p = (params or CostParams()).to_c()
    return float(lib().ft_cost_v1_oneshot(world, nbytes, C.byref(p)))


def cost_v1_nvls(world: int, nbytes: int, params: CostParams | None = None) -> float:
    p = (params or CostParams()).to_c()
    return float(lib().ft_cost_v1_nvls(world, nbytes, C.byref(p)))


def pick_algorithm(world: int, nbytes: int, params: CostParams | None = None, allow_oneshot: bool = True,
                   allow_nvls: bool = True) -> tuple[str, Shape, float]:
    """(algorithm, shape, predicted microseconds) for a message of ``nbytes``."""
    p = (params or CostParams()).to_c()
    w = (C.c_int * 64)()
    lonely, ring, us = C.c_int(), C.c_int(), C.c_double()
    algo = C.create_string_buffer(32)
    k = lib().ft_pick_algorithm(world, nbytes, C.byref(p), int(allow_oneshot), int(allow_nvls), w, 64,
                                C.byref(lonely), C.byref(ring), algo, 32, C.byref(us))
    return algo.value.decode(), Shape(tuple(w[i] for i in range(k)), lonely.value, bool(ring.value)), us.value


# ---- configuration ----------------------------------------------------------------------
def parse_topo(topo: str | None, lonely: str | None, world: int) -> tuple[Shape, bool]:
    """``FT_TOPO`` / ``FT_LONELY`` syntax -> (shape, is_auto); raises on an invalid layout."""
    w = (C.c_int * 64)()
    nw, l, ring, is_auto = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    err = C.create_string_buffer(512)
    code = lib().ft_parse_topo((topo or "").encode(), (lonely or "").encode(), world, w, 64, C.byref(nw), C.byref(l),
                               C.byref(ring), C.byref(is_auto), err, 512)
    if code:
        raise FlexTreeError(code, err.value.decode())
    return Shape(tuple(w[i] for i in range(nw.value)), l.value, bool(ring.value)), bool(is_auto.value)


def shape_from_env(world: int) -> tuple[Shape, bool]:
    return parse_topo(os.environ.get("FT_TOPO"), os.environ.get("FT_LONELY"), world)


# ---- planner ----------------------------------------------------------------------------
def validate_shape(world: int, shape: Shape) -> str:
    """Empty string when executable, else the reason."""
    err = C.create_string_buffer(512)
    lib().ft_validate_shape(world, *shape.c_args(), err, 512)
    return err.value.decode()


def plan_check(world: int, shape: Shape) -> str:
    """Static race check of the in-place schedule: empty string when race-free."""
    err = C.create_string_buffer(1024)
    lib().ft_plan_check(world, *shape.c_args(), err, 1024)
    return err.value.decode()


def dev_plan_check(world: int, shape: Shape, rank: int) -> str:
    """Descriptor check of ``rank``'s device table (what the communicator verifies before upload):
    empty string when every index, block id, fan-in, source rank and rendezvous mask is in range."""
    err = C.create_string_buffer(1024)
    lib().ft_dev_plan_check(world, *shape.c_args(), rank, err, 1024)
    return err.value.decode()


def plan_num_stages(world: int, shape: Shape) -> int:
    return lib().ft_plan_num_stages(world, *shape.c_args())


def plan_max_fanin(world: int, shape: Shape) -> int:
    return lib().ft_plan_max_fanin(world, *shape.c_args())


def plan_traffic(world: int, shape: Shape, count: int, block_elems: int = 0) -> int:
    return int(lib().ft_plan_traffic(world, *shape.c_args(), count, block_elems))


def describe(world: int, shape: Shape, rank: int, count: int = 0, block_elems: int = 0) -> str:
    return text_call(lib().ft_plan_describe, world, *shape.c_args(), rank, count, block_elems)


def context(world: int, rank: int, count: int, dtype: torch.dtype = torch.float32, lonely: int = 0) -> dict:
    """The per-call quantities of the reference's FlexTree_Context (mpi_mod.hpp:776-801) as a dict:
    num_nodes, node_label, num_lonely, data_size, num_split, split_size, data_size_aligned, type_size, has_lonely."""
    line = text_call(lib().ft_context_describe, world, rank, lonely, count, ft_dtype(dtype))
    return {k: int(v) for k, v in (kv.split("=") for kv in line.strip().split(", "))}


def plan_json(world: int, shape: Shape) -> dict:
    return json.loads(text_call(lib().ft_plan_json, world, *shape.c_args(), cap=1 << 20))


# ---- CPU executors ----------------------------------------------------------------------
def run_plan_snapshot(shape: Shape, bufs: Sequence[torch.Tensor], op: str = "sum", block_elems: int = 0,
                      phase: str = "all") -> None:
    """All ranks in this thread, in place on ``bufs[rank]`` (CPU tensors).  ``phase`` runs one half of
    the plan alone: "reduce_scatter" (afterwards :func:`rs_holders` says who holds which block) or
    "all_gather"."""
    world = len(bufs)
    ptrs = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    half = plan_num_stages(world, shape) // 2
    begin, end = {"all": (0, -1), "reduce_scatter": (0, half), "all_gather": (half, -1)}[phase]
    check(lib().ft_run_plan_snapshot_range(world, *shape.c_args(), OPS[op], ft_dtype(bufs[0].dtype), ptrs, bufs[0].numel(),
                                           block_elems, begin, end), f"shape {shape} for world {world}")


def rs_holders(world: int, shape: Shape) -> list[list[int]]:
    """``holders[b]`` = ranks whose block ``b`` is complete after the reduce-scatter half alone.  In a
    plain tree every block has one holder; with lonely ranks a lonely rank shares its holder's blocks."""
    masks = (C.c_uint64 * world)()
    check(lib().ft_plan_rs_holders(world, *shape.c_args(), masks), f"shape {shape} for world {world}")
    return [[r for r in range(world) if masks[b] >> r & 1] for b in range(world)]


def owned_blocks(world: int, shape: Shape, rank: int) -> list[int]:
    """Blocks that ``rank`` holds complete after a reduce-scatter, and must hold valid before an all-gather."""
    return [b for b, hs in enumerate(rs_holders(world, shape)) if rank in hs]


def block_elems_for(count: int, world: int, elem_size: int) -> int:
    """Elements per block as the GPU communicator cuts a tensor (the library's own arithmetic): ceil(count / world)
    rounded up to whole 16-byte vectors, and to whole multiples of 512 bytes once a block reaches 64 KiB;
    block b covers [b * B, min((b + 1) * B, count))."""
    return int(lib().ft_block_elems(count, world, elem_size))


class CpuWorld:
    """Thread-per-rank world running the device protocol (epoch flags, bounded waits) on the host."""

    def __init__(self, world: int, timeout_s: float = 5.0):
        self.world = world
        self._h = lib().ft_cpu_world_create(world, timeout_s)
        if not self._h:
            raise ValueError("bad world size")

    def close(self):
        if self._h:
            lib().ft_cpu_world_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def allreduce_rank(self, rank: int, shape: Shape, recv: torch.Tensor, send: torch.Tensor | None = None,
                       op: str = "sum", block_elems: int = 0, fault=(0, -1, 0)) -> tuple[int, int, int]:
        """One rank's call (blocking); returns (status, rendezvous index, peer)."""
        st = (C.c_int * 3)()
        lib().ft_cpu_allreduce(self._h, rank, *shape.c_args(), OPS[op], ft_dtype(recv.dtype),
                               send.data_ptr() if send is not None else None, recv.data_ptr(), recv.numel(),
                               block_elems, fault[0], fault[1], fault[2], st)
        return st[0], st[1], st[2]

    def phase_rank(self, rank: int, shape: Shape, buf: torch.Tensor, phase: str, op: str = "sum",
                   block_elems: int = 0) -> tuple[int, int, int]:
        """One rank's call of one half of the plan, in place: ``phase`` "reduce_scatter" or "all_gather"."""
        st = (C.c_int * 3)()
        lib().ft_cpu_phase(self._h, rank, *shape.c_args(), OPS[op], ft_dtype(buf.dtype), buf.data_ptr(), buf.numel(),
                           block_elems, {"reduce_scatter": 1, "all_gather": 2}[phase], st)
        return st[0], st[1], st[2]

    def allreduce(self, shape: Shape, bufs: Sequence[torch.Tensor], op: str = "sum", block_elems: int = 0,
                  fault=(0, -1, 0)) -> list[tuple[int, int, int]]:
        """Run every rank on its own thread, in place on ``bufs``; returns per-rank status."""
        out: list = [None] * self.world

        def work(r):
            out[r] = self.allreduce_rank(r, shape, bufs[r], None, op, block_elems, fault)

        ts = [threading.Thread(target=work, args=(r,)) for r in range(self.world)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        return out


class ProcWorld:
    """This process as one rank of a world of ordinary processes on one host (launched like an MPI job, no MPI
    library): control state in a POSIX shared-memory segment named after ``session`` (unique per job), data
    pulled straight out of the peers' buffers with ``process_vm_readv`` (messages up to 16 KiB through the
    segment).  ``join`` is collective; rank / world / session default to FT_RANK / FT_WORLD / FT_SESSION,
    else RANK / WORLD_SIZE / MASTER_PORT (what ``torch.distributed.run`` sets)."""

    def __init__(self, session: str | None = None, rank: int | None = None, world: int | None = None, timeout_s: float = 30.0):
        env = os.environ
        rank = int(env.get("FT_RANK") or env["RANK"]) if rank is None else rank
        world = int(env.get("FT_WORLD") or env["WORLD_SIZE"]) if world is None else world
        session = session or env.get("FT_SESSION") or env["MASTER_PORT"]
        err = C.create_string_buffer(256)
        self._h = lib().ft_proc_world_join(str(session).encode(), rank, world, timeout_s, err, 256)
        if not self._h:
            raise FlexTreeError(9, err.value.decode())
        self.rank, self.world = rank, world

    device = torch.device("cpu")   # the surface FlexTreeDDP expects of a communicator: alloc, all_reduce, world, rank, device

    def all_reduce(self, tensor: torch.Tensor, shape: Shape | str | None = None, op: str = "sum", out: torch.Tensor | None = None,
                   **_ignored) -> torch.Tensor:
        """All-reduce a contiguous CPU tensor across the processes (in place unless ``out`` is given).
        ``op``: "sum", "band" or "avg" (floating types; the sum divided by the world size)."""
        dst = tensor if out is None else out
        if tensor.is_cuda or not tensor.is_contiguous() or not dst.is_contiguous() or dst.numel() != tensor.numel():
            raise ValueError("needs contiguous CPU tensors of equal size")
        if op == "avg":
            self.all_reduce(tensor, shape, "sum", out)
            return dst.div_(self.world)
        if isinstance(shape, str):
            shape = Shape.parse(shape)
        shp = shape or shape_from_env(self.world)[0]
        st = (C.c_int * 3)()
        code = lib().ft_proc_allreduce(self._h, *shp.c_args(), OPS[op], ft_dtype(tensor.dtype),
                                       None if dst is tensor else tensor.data_ptr(), dst.data_ptr(), tensor.numel(), st)
        if code:
            raise FlexTreeError(code, f"rendezvous {st[1]}, peer {st[2]}: {lib().ft_proc_last_error(self._h).decode()}")
        return dst

    def _phase(self, tensor: torch.Tensor, shape, op: str, phase: int) -> Shape:
        if tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("needs a contiguous CPU tensor")
        shp = shape or shape_from_env(self.world)[0]
        st = (C.c_int * 3)()
        code = lib().ft_proc_phase(self._h, *shp.c_args(), OPS[op], ft_dtype(tensor.dtype), tensor.data_ptr(), tensor.numel(), phase, st)
        if code:
            raise FlexTreeError(code, f"rendezvous {st[1]}, peer {st[2]}: {lib().ft_proc_last_error(self._h).decode()}")
        return shp

    def reduce_scatter(self, tensor: torch.Tensor, shape: Shape | None = None, op: str = "sum") -> list[torch.Tensor]:
        """Reduce-scatter half alone, in place; returns views of the block(s) this rank then holds complete
        (block b covers elements [b * B, (b + 1) * B), B = ceil(numel / world)).  ``op="avg"`` divides those
        blocks by the world size."""
        if isinstance(shape, str):
            shape = Shape.parse(shape)
        shp = self._phase(tensor, shape, "sum" if op == "avg" else op, 1)
        B = -(-tensor.numel() // self.world)
        flat = tensor.view(-1)
        mine = [flat[min(flat.numel(), b * B):min(flat.numel(), (b + 1) * B)] for b in owned_blocks(self.world, shp, self.rank)]
        if op == "avg":
            for v in mine:
                v.div_(self.world)
        return mine

    def all_gather(self, tensor: torch.Tensor, shape: Shape | None = None) -> torch.Tensor:
        """All-gather half alone: every rank's own blocks are taken as final and copied to all the others."""
        if isinstance(shape, str):
            shape = Shape.parse(shape)
        self._phase(tensor, shape, "sum", 2)
        return tensor

    def profile_phases(self, tensor: torch.Tensor, shape: Shape | None = None, iters: int = 5) -> dict:
        """Host time (ms, this rank, barrier to return) of the two halves, each issued as a call of its own: what the
        reference's SHOW_TIME switch logs around its reduce-scatter and all-gather loops (mpi_mod.hpp:31-35,
        :1597-1599, :1645-1647).  The tensor's contents are reduced ``iters`` times."""
        import time
        acc = [0.0, 0.0]
        for _ in range(iters):
            self.barrier()
            t0 = time.perf_counter()
            self.reduce_scatter(tensor, shape)
            t1 = time.perf_counter()
            self.all_gather(tensor, shape)
            t2 = time.perf_counter()
            acc[0] += (t1 - t0) * 1e3 / iters
            acc[1] += (t2 - t1) * 1e3 / iters
        return {"reduce_scatter_ms": acc[0], "all_gather_ms": acc[1]}

    def heap_create(self, nbytes: int):
        """Collective, once: every rank gets a shared segment of ``nbytes`` that all the others map.  Tensors from
        :meth:`alloc` are then reduced in place with plain loads from the peers' mappings (no system call, no
        copy), as long as every rank allocates in the same order."""
        if lib().ft_proc_heap_create(self._h, nbytes):
            raise FlexTreeError(9, lib().ft_proc_last_error(self._h).decode())

    def alloc(self, shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """CPU tensor inside this rank's shared heap segment (call :meth:`heap_create` first)."""
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = max(1, n * torch.empty((), dtype=dtype).element_size())
        ptr = lib().ft_proc_alloc(self._h, nbytes)
        if not ptr:
            raise MemoryError("the process world's heap is exhausted (or heap_create was not called)")
        t = torch.frombuffer((C.c_char * nbytes).from_address(ptr), dtype=dtype, count=n).view(shape)
        t._ft_owner = self   # the mapping lives as long as the world
        return t

    def free(self, tensor: torch.Tensor):
        check(lib().ft_proc_free(self._h, tensor.data_ptr()), "not a tensor from alloc()")

    def symmetric(self, tensor: torch.Tensor) -> bool:
        """Collective check that ``tensor`` sits at the same heap offset on every rank."""
        return bool(lib().ft_proc_heap_symmetric(self._h, tensor.data_ptr()))

    def barrier(self):
        check(lib().ft_proc_barrier(self._h), "barrier")

    def close(self):
        if self._h:
            lib().ft_proc_world_leave(self._h)
            self._h = None

    def __del__(self):
        self.close()
