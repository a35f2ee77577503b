"""FlexTree communicator: all-reduce over NVLink peer memory with hand-written kernels.

``FlexTreeComm`` is the per-process object (one process per GPU).  ``torch.distributed`` is
used only as the bootstrap that carries memory handles between ranks; the data path is
``libflextree.so``'s kernels reading peers' symmetric heaps directly.

    comm = FlexTreeComm(heap_bytes=1 << 30)          # after dist.init_process_group
    g = comm.alloc((n,), torch.bfloat16)             # tensor in the symmetric heap: zero-copy
    comm.all_reduce(g, shape="auto")                 # picks one-shot / tree / NVLS per size
    comm.all_reduce(any_cuda_tensor, shape="2*4")    # staged through internal slots

``LocalWorld`` puts all ranks in one process: on several GPUs (micro-benchmarks), or on ONE
GPU with the ranks emulated stage by stage in stream order (tests without a multi-GPU box).

Reference counterpart: ``MPI_Allreduce_FT`` and its FT_TOPO / FT_LONELY configuration
(allreduce_over_mpi/mpi_mod.hpp:1419-1486, :1723-1778).
"""
from __future__ import annotations

import ctypes as C
import os
import uuid
from typing import Sequence

import torch

from .._lib import Choice, FlexTreeError, OPS, lib
from ..ops.reduce import ft_dtype
from ..utils import log
from . import planner
from .planner import Shape

ALGOS = {"auto": 0, "staged": 1, "oneshot": 2, "nvls": 3, "hybrid": 4, "ll": 5, "push": 6, "nvls1": 9}
LL_MAX_BYTES = 256 << 10
CANARY_BYTES, CANARY_BYTE = 256, 0xA5
MEM_IPC, MEM_VMM = 0, 1


class _Span:
    """Exposes raw device memory to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device, owner=None) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    flat = torch.as_tensor(_Span(ptr, max(nbytes, 1), owner), device=device)
    return flat[:nbytes].view(dtype).view(*shape)


def _as_shape(shape, world) -> Shape | None:
    if shape is None or isinstance(shape, Shape):
        return shape
    if isinstance(shape, str):
        return None if shape in ("auto", "") else Shape.parse(shape)
    return Shape(tuple(int(x) for x in shape))


class _CommBase:
    """Shared by process-per-GPU and in-process communicators: one native ft_comm handle."""

    def __init__(self):
        self._h = C.c_void_p()
        self.rank = 0
        self.world = 1
        self.device = torch.device("cuda", 0)
        self.default_shape: Shape | None = None
        self.auto = True
        self.has_nvls = False
        self._policy = None   # (world, handle) of a free-standing native policy, see _policy_handle()
        self.ll_auto_max = int(os.environ.get("FT_LL_MAX_BYTES", 8 << 10))
        self._heap_range = None
        self._poisoned = False
        self._nvtx = os.environ.get("FT_NVTX", "0") == "1"   # NVTX range around every call (for timeline tools)
        # guard words behind every alloc() (debugging aid, FT_CANARY=1 or enable_canaries())
        self._canaries: list | None = [] if os.environ.get("FT_CANARY", "0") == "1" else None

    # -- errors
    def _check(self, code: int):
        if code:
            raise FlexTreeError(code, lib().ft_comm_last_error(self._h).decode())

    def _create(self, rank, world, device_index, heap_bytes, staging_bytes, mem_kind):
        self.rank, self.world = rank, world
        self.device = torch.device("cuda", device_index)
        self.heap_bytes, self.staging_bytes = heap_bytes, staging_bytes
        code = lib().ft_comm_create(rank, world, device_index, heap_bytes, staging_bytes, mem_kind, C.byref(self._h))
        return code

    def _configure_from_env(self):
        shape, is_auto = planner.shape_from_env(self.world)
        self.auto = is_auto or not (os.environ.get("FT_TOPO") or os.environ.get("FT_LONELY"))
        self.default_shape = None if self.auto else shape
        if os.environ.get("FT_TIMEOUT_MS"):
            self.set_timeout_ms(float(os.environ["FT_TIMEOUT_MS"]))
        if os.environ.get("FT_MAX_LANES"):
            self.set_max_lanes(int(os.environ["FT_MAX_LANES"]))
        lib().ft_comm_set_ll_max(self._h, self.ll_auto_max)
        env = os.environ
        if any(env.get(k) for k in ("FT_NVLS_THREADS", "FT_NVLS_UNROLL", "FT_NVLS_WEAK", "FT_NVLS_MAX_LANES", "FT_NVLS_STRIPE")):
            self.set_nvls_config(threads=int(env.get("FT_NVLS_THREADS", 0)), unroll=int(env.get("FT_NVLS_UNROLL", 0)),
                                 weak=int(env["FT_NVLS_WEAK"]) if env.get("FT_NVLS_WEAK") else None,
                                 max_lanes=int(env["FT_NVLS_MAX_LANES"]) if env.get("FT_NVLS_MAX_LANES") else None,
                                 stripe_bytes=int(env["FT_NVLS_STRIPE"]) if env.get("FT_NVLS_STRIPE") else None)
        if os.environ.get("FT_NVLS_CTAS_PER_SM"):
            lib().ft_comm_set_nvls_ctas_per_sm(self._h, int(os.environ["FT_NVLS_CTAS_PER_SM"]))

    # -- knobs
    def set_timeout_ms(self, ms: float):
        lib().ft_comm_set_timeout_ms(self._h, ms)

    def set_max_lanes(self, lanes: int):
        lib().ft_comm_set_max_lanes(self._h, lanes)

    def set_oneshot_max(self, nbytes: int):
        lib().ft_comm_set_oneshot_max(self._h, nbytes)

    def set_nvls_config(self, threads: int = 0, unroll: int = 0, weak: int | None = None, max_lanes: int | None = None,
                        stripe_bytes: int | None = None):
        """Launch shape of the NVLS kernels: threads per CTA, 16-byte vectors in flight per thread (2/4/8), the
        ``.weak`` instruction form, a cap on the CTAs per launch (0: one per SM) and, for the all-reduce, ownership by
        round-robin stripes of ``stripe_bytes`` instead of one block per rank (0).  Arguments left at their
        defaults keep the current setting.  Environment: FT_NVLS_THREADS / _UNROLL / _WEAK / _MAX_LANES / _STRIPE."""
        self._check(lib().ft_comm_set_nvls_config(self._h, threads, unroll, -1 if weak is None else int(weak),
                                                  -1 if max_lanes is None else int(max_lanes),
                                                  C.c_size_t(-1).value if stripe_bytes is None else int(stripe_bytes)))

    def set_hybrid(self, byte_fraction: float, lane_fraction: float):
        """Split used by algo="hybrid": share of each block reduced in the switch, share of the CTAs doing it."""
        lib().ft_comm_set_hybrid(self._h, byte_fraction, lane_fraction)

    # -- symmetric heap
    def alloc(self, shape, dtype=torch.float32) -> torch.Tensor:
        """Tensor inside the symmetric heap (same offset on every rank when every rank allocates
        in the same order).  All-reduce on such a tensor is in place and copy-free."""
        if isinstance(shape, int):
            shape = (shape,)
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        ptr = lib().ft_comm_alloc(self._h, nbytes)
        if not ptr:
            raise MemoryError(f"symmetric heap exhausted ({self.heap_bytes} bytes); pass a larger heap_bytes")
        t = tensor_from_ptr(ptr, shape, dtype, self.device, owner=self)
        if self._canaries is not None:
            gptr = lib().ft_comm_alloc(self._h, CANARY_BYTES)
            if not gptr:
                raise MemoryError("symmetric heap exhausted while placing a guard block")
            guard = tensor_from_ptr(gptr, (CANARY_BYTES,), torch.uint8, self.device, owner=self)
            guard.fill_(CANARY_BYTE)
            self._canaries.append((guard, f"{tuple(shape)} {dtype} at heap offset {ptr - (lib().ft_comm_heap_base(self._h) or 0)}", ptr))
        return t

    def free(self, tensor: torch.Tensor):
        """Give a tensor from :meth:`alloc` back to the heap (it must no longer be used).  Like alloc(), every
        rank has to do this in the same order for later allocations to stay symmetric."""
        ptr = tensor.data_ptr()
        self._check(lib().ft_comm_free(self._h, ptr))
        if self._canaries:   # the guard block behind it goes too
            for k, (guard, what, owner_ptr) in enumerate(self._canaries):
                if owner_ptr == ptr:
                    lib().ft_comm_free(self._h, guard.data_ptr())
                    del self._canaries[k]
                    break

    @property
    def heap_free_bytes(self) -> int:
        """Largest tensor :meth:`alloc` could hand out right now."""
        return int(lib().ft_comm_heap_free_bytes(self._h))

    def free_all(self):
        """Forget every alloc() (tensors handed out before must no longer be used)."""
        lib().ft_comm_alloc_reset(self._h)
        if self._canaries is not None:
            self._canaries = []

    def enable_canaries(self, on: bool = True):
        """Place a 256-byte guard block of a known pattern behind every later alloc().  Kernels address a
        heap tensor by block and lane offsets computed from its length; a wrong offset that runs past the
        tensor lands in the guard, and :meth:`check_canaries` reports it.  (compute-sanitizer's memcheck does
        the same job where it is available; this works everywhere and across ranks, since peers write into
        this heap too.)"""
        self._canaries = [] if on else None

    def check_canaries(self, synchronize: bool = True) -> int:
        """Raise if any guard block was overwritten; returns the number of guards checked."""
        if self._canaries is None:
            return 0
        if synchronize:
            torch.cuda.synchronize(self.device)
        hit = [what for guard, what, _ in self._canaries if not bool((guard == CANARY_BYTE).all())]
        if hit:
            raise FlexTreeError(8, f"rank {self.rank}: memory behind these heap tensors was overwritten: " + "; ".join(hit))
        return len(self._canaries)

    def in_heap(self, t: torch.Tensor) -> bool:
        if self._heap_range is None:
            base = lib().ft_comm_heap_base(self._h) or 0
            self._heap_range = (base, base + lib().ft_comm_heap_bytes(self._h))
        p = t.data_ptr()   # in place only from a 16-byte boundary (the kernels use vector loads there)
        return self._heap_range[0] <= p and p + t.numel() * t.element_size() <= self._heap_range[1] and p % 16 == 0

    # -- selection
    def _policy_handle(self):
        """The native selection policy: the communicator's own once it exists, else a free-standing one
        for this world size loaded from the same calibration file (host-only use and tests)."""
        if self._h:
            h = lib().ft_comm_policy(self._h)
            if h:
                return h
        if self._policy is None or self._policy[0] != self.world:
            h = lib().ft_policy_create(self.world)
            err = C.create_string_buffer(256)
            lib().ft_policy_load(h, None, err, 256)
            self._policy = (self.world, h)
        return self._policy[1]

    def choose(self, nbytes: int, in_heap: bool, dtype: torch.dtype) -> tuple[str, Shape]:
        """Algorithm and shape for a message: the measured winner for this world and size from the calibration
        table, else the calibrated cost model.  This asks the same native policy object that
        ``ft_allreduce(FT_ALGO_AUTO)``, ``MPI_Allreduce_FT`` and ``ft_bench`` use (csrc/planner/policy.hpp)."""
        nvls_ok = self.has_nvls and in_heap and dtype in (torch.float32, torch.bfloat16, torch.float16) and nbytes % 16 == 0
        nvls1_ok = self.has_nvls and dtype in (torch.float32, torch.bfloat16, torch.float16)
        out = Choice()
        code = lib().ft_policy_choose(self._policy_handle(), nbytes, int(bool(in_heap)), int(bool(nvls_ok)),
                                      int(self.staging_bytes), int(self.ll_auto_max), int(bool(nvls1_ok)), C.byref(out))
        if code:
            raise FlexTreeError(code, "selection policy")
        name = out.algo_name.decode()
        if name == "hybrid":
            name = f"hybrid-{out.hybrid_bytes:g}-{out.hybrid_lanes:g}"
        return name, Shape(tuple(out.widths[i] for i in range(out.nw)), out.lonely, bool(out.ring))

    # -- the collective
    def all_reduce(self, tensor: torch.Tensor, op: str = "sum", shape=None, algo: str = "auto", scale: float = 1.0,
                   out: torch.Tensor | None = None, stream: torch.cuda.Stream | None = None) -> torch.Tensor:
        """All-reduce ``tensor`` across the world on ``stream`` (default: current stream).

        ``op``: "sum", "band" or "avg" (sum scaled by 1/world, floating types).  ``shape``: None/"auto"
        (cost model, or FT_TOPO/FT_LONELY when set), a :class:`Shape`, or text such as "2*4", "2*2+1",
        "ring8".  ``out``: result tensor (default in place).  Tensors that live in the symmetric
        heap are reduced in place with no copy; others are staged through internal slots (and
        split when larger than one slot)."""
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("all_reduce needs a contiguous CUDA tensor")
        if tensor.device != self.device or (out is not None and out.device != self.device):
            raise ValueError(f"tensor on {tensor.device}, communicator on {self.device}")
        if self._poisoned:
            raise FlexTreeError(5, "a device-side wait timed out earlier: the ranks' call counters no longer agree, "
                                   "rebuild the communicator (see parallel/elastic.py for a smaller world)")
        if op == "avg":
            op, scale = "sum", scale / self.world
        dst = tensor if out is None else out
        if dst.numel() != tensor.numel() or dst.dtype != tensor.dtype or not dst.is_contiguous():
            raise ValueError("out must match the input")
        shp = _as_shape(shape, self.world)
        if shp is None and not self.auto:
            shp = self.default_shape
        a = ALGOS[algo]
        nbytes = tensor.numel() * tensor.element_size()
        # algo "auto" without a shape: the native policy decides inside ft_allreduce (see choose())
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        dt = ft_dtype(tensor.dtype)

        def call(src_ptr, dst_ptr, count):
            if shp is None:
                arr, nw, lonely, ring = None, 0, 0, 0
            else:
                arr, nw, lonely, ring = shp.c_args()
            self._check(lib().ft_allreduce(self._h, src_ptr, dst_ptr, count, dt, OPS[op], arr, nw, lonely, ring, a,
                                           float(scale), C.c_void_p(st)))

        nvtx = self._nvtx
        if nvtx:
            torch.cuda.nvtx.range_push(f"flextree.all_reduce {nbytes}B {algo if a else 'auto'}")
        with torch.cuda.device(self.device):
            src_ptr = None if dst.data_ptr() == tensor.data_ptr() else tensor.data_ptr()
            call(src_ptr, dst.data_ptr(), tensor.numel())   # tensors larger than a staging slot are split natively
        if nvtx:
            torch.cuda.nvtx.range_pop()
        return dst

    def all_reduce_host(self, src: torch.Tensor, out: torch.Tensor | None = None, op: str = "sum", shape=None,
                        algo: str = "auto", scale: float = 1.0, stream: torch.cuda.Stream | None = None) -> torch.Tensor:
        """All-reduce of a tensor in (pinned) HOST memory, the form the reference's ``MPI_Allreduce_FT`` takes
        (allreduce_over_mpi/mpi_mod.hpp:1723-1778 knows host buffers only).  The message is pipelined through
        three chunk buffers of the symmetric heap: the copy in of chunk k+1, the NVLink all-reduce of chunk k and
        the copy out of chunk k-1 overlap.  Collective: every rank calls it.  The result (``out``, default in
        place) is complete once ``stream`` (default: the current stream) has been synchronised."""
        dst = src if out is None else out
        for t in (src, dst):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("all_reduce_host needs contiguous CPU tensors (pinned for full speed)")
        if dst.numel() != src.numel() or dst.dtype != src.dtype:
            raise ValueError("out must match the input")
        if self._poisoned:
            raise FlexTreeError(5, "a device-side wait timed out earlier: rebuild the communicator")
        if op == "avg":
            op, scale = "sum", scale / self.world
        shp = _as_shape(shape, self.world)
        if shp is None and not self.auto:
            shp = self.default_shape
        arr, nw, lonely, ring = (None, 0, 0, 0) if shp is None else shp.c_args()
        with torch.cuda.device(self.device):
            st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
            self._check(lib().ft_allreduce_host(self._h, None if dst.data_ptr() == src.data_ptr() else src.data_ptr(), dst.data_ptr(),
                                                src.numel(), ft_dtype(src.dtype), OPS[op], arr, nw, lonely, ring, ALGOS[algo],
                                                float(scale), C.c_void_p(st)))
        return dst

    # -- the two halves of the staged plan as collectives of their own
    def _phase_shape(self, shape) -> Shape:
        shp = _as_shape(shape, self.world)
        if shp is None:
            shp = self.default_shape if not self.auto and self.default_shape is not None else Shape.flat(self.world)
        return shp

    def block_range(self, tensor: torch.Tensor, block: int) -> tuple[int, int]:
        """Element range [lo, hi) of ``block`` when ``tensor`` is cut for a collective (``world`` blocks of
        whole 16-byte vectors; trailing blocks may be short or empty)."""
        n = tensor.numel()
        B = planner.block_elems_for(n, self.world, tensor.element_size())
        return min(n, block * B), min(n, (block + 1) * B)

    def owned_blocks(self, shape=None) -> list[int]:
        """Blocks this rank holds complete after :meth:`reduce_scatter` with ``shape`` (block = rank for
        trees, rank + 1 for the ring)."""
        return planner.owned_blocks(self.world, self._phase_shape(shape), self.rank)

    def _phase(self, tensor: torch.Tensor, gather: bool, op: str, shape, scale: float, stream):
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("needs a contiguous CUDA tensor")
        if tensor.device != self.device:
            raise ValueError(f"tensor on {tensor.device}, communicator on {self.device}")
        if self.world > 1 and not self.in_heap(tensor):
            raise ValueError("reduce_scatter / all_gather work in place on a tensor from comm.alloc()")
        if self._poisoned:
            raise FlexTreeError(5, "a device-side wait timed out earlier: rebuild the communicator")
        shp = self._phase_shape(shape)
        arr, nw, lonely, ring = shp.c_args()
        st = C.c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)
        with torch.cuda.device(self.device):
            if gather:
                self._check(lib().ft_all_gather(self._h, tensor.data_ptr(), tensor.numel(), ft_dtype(tensor.dtype), arr, nw, lonely,
                                                ring, st))
            else:
                self._check(lib().ft_reduce_scatter(self._h, tensor.data_ptr(), tensor.numel(), ft_dtype(tensor.dtype), OPS[op], arr,
                                                    nw, lonely, ring, float(scale), st))
        return shp

    def reduce_scatter(self, tensor: torch.Tensor, op: str = "sum", shape=None, scale: float = 1.0,
                       stream: torch.cuda.Stream | None = None) -> list[torch.Tensor]:
        """Reduce-scatter half of the staged all-reduce, in place on a heap tensor.  Returns views of the
        blocks this rank now holds complete (one block; the rest of ``tensor`` holds partial sums)."""
        if op == "avg":
            op, scale = "sum", scale / self.world
        shp = self._phase(tensor, False, op, shape, scale, stream)
        flat = tensor.view(-1)
        return [flat[slice(*self.block_range(tensor, b))] for b in planner.owned_blocks(self.world, shp, self.rank)]

    def all_gather(self, tensor: torch.Tensor, shape=None, stream: torch.cuda.Stream | None = None) -> torch.Tensor:
        """All-gather half: every rank's own blocks (:meth:`owned_blocks`) are taken as final and copied to
        every other rank, in place on a heap tensor."""
        self._phase(tensor, True, "sum", shape, 1.0, stream)
        return tensor

    def profile_phases(self, tensor: torch.Tensor, shape=None, op: str = "sum", iters: int = 5) -> dict:
        """Device time (ms, this rank) of the two halves of the staged all-reduce on a heap tensor, each
        issued as a call of its own between CUDA events: what the reference's SHOW_TIME switch logs with
        MPI_Wtime around its reduce-scatter and all-gather loops (allreduce_over_mpi/mpi_mod.hpp:31-35,
        :1597-1599, :1645-1647).  The tensor's contents are reduced ``iters + 1`` times."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        acc = [0.0, 0.0]
        self.reduce_scatter(tensor, op=op, shape=shape)     # warm-up: plan upload, first touch
        self.all_gather(tensor, shape=shape)
        for _ in range(iters):
            ev[0].record()
            self.reduce_scatter(tensor, op=op, shape=shape)
            ev[1].record()
            self.all_gather(tensor, shape=shape)
            ev[2].record()
            ev[2].synchronize()
            acc[0] += ev[0].elapsed_time(ev[1]) / iters
            acc[1] += ev[1].elapsed_time(ev[2]) / iters
        return {"reduce_scatter_ms": acc[0], "all_gather_ms": acc[1], "shape": str(self._phase_shape(shape))}

    # -- health
    def status(self) -> dict:
        """Status block written by device-side bounded waits (call after synchronising)."""
        out = (C.c_int * 5)()
        lib().ft_comm_status(self._h, out)
        return {"code": out[0], "rendezvous": out[1], "peer": out[2], "lane": out[3], "calls": out[4]}

    def stats(self) -> dict:
        """Calls and message bytes so far per algorithm as resolved at launch (host-side counters), e.g.
        ``{"nvls": {"calls": 12, "bytes": 3221225472}, "ll": {...}, "reduce_scatter": {...}}``."""
        calls, nbytes = (C.c_uint64 * 10)(), (C.c_uint64 * 10)()
        self._check(lib().ft_comm_stats(self._h, calls, nbytes))
        names = {v: k for k, v in ALGOS.items()}
        names.update({7: "reduce_scatter", 8: "all_gather"})
        return {names[k]: {"calls": int(calls[k]), "bytes": int(nbytes[k])} for k in range(1, 10) if calls[k]}

    def check(self, synchronize: bool = True):
        """Raise if a device-side wait timed out (a peer never arrived)."""
        if synchronize:
            torch.cuda.synchronize(self.device)
        s = self.status()
        if s["code"]:
            lib().ft_comm_clear_status(self._h)
            self._poisoned = self.world > 1
            raise FlexTreeError(s["code"], f"rank {self.rank}: wait on rank {s['peer']} at rendezvous {s['rendezvous']} (lane {s['lane']})")

    def wait_probe(self, peer: int, timeout_ms: float = 1.0):
        """Launch a kernel that waits ``timeout_ms`` for a signal from ``peer`` that never comes."""
        st = torch.cuda.current_stream(self.device).cuda_stream
        self._check(lib().ft_comm_wait_probe(self._h, peer, timeout_ms, C.c_void_p(st)))

    def close(self):
        """Unmap the heaps and free the communicator.  Tensors handed out by :meth:`alloc` point into the
        heap: they must not be touched afterwards (drop them first)."""
        if self._h:
            try:
                log.debug(f"closing; usage {self.stats()}", self.rank)
            except Exception:  # noqa: BLE001 - a summary line must never get in the way of teardown
                pass
            self._canaries = None if self._canaries is None else []
            lib().ft_comm_destroy(self._h)
            self._h = C.c_void_p()
        if self._policy is not None:
            lib().ft_policy_destroy(self._policy[1])
            self._policy = None

    def __del__(self):
        try:
            self.close(False) if isinstance(self, FlexTreeComm) else self.close()
        except Exception:
            pass


class FlexTreeComm(_CommBase):
    """One rank of a multi-process world (launch with torchrun, one process per GPU)."""

    def __init__(self, group=None, heap_bytes: int = 1 << 30, staging_bytes: int = 64 << 20, mem: str | None = None,
                 nvls: bool | None = None, device: int | None = None):
        super().__init__()
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("init torch.distributed first (it only carries the memory handles)")
        self.group = group
        self._check_symmetric = os.environ.get("FT_CHECK_SYMMETRIC", "0") == "1"
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        dev = device if device is not None else int(os.environ.get("LOCAL_RANK", rank % max(1, torch.cuda.device_count())))
        torch.cuda.set_device(dev)
        mem = (mem or os.environ.get("FT_MEM", "auto")).lower()
        kinds = {"auto": [MEM_VMM, MEM_IPC], "vmm": [MEM_VMM], "ipc": [MEM_IPC]}[mem]
        last = None
        for kind in kinds:
            code = self._create(rank, world, dev, heap_bytes, staging_bytes, kind)
            ok = self._exchange(kind) if code == 0 else False
            oks = [None] * world
            dist.all_gather_object(oks, bool(ok), group=group)
            if all(oks):
                break
            last = lib().ft_comm_last_error(self._h).decode() if self._h else "create failed"
            log.warn(f"symmetric memory kind {kind} unavailable ({last}); trying the next one", rank)
            self.close()
        else:
            raise FlexTreeError(9, f"no usable symmetric memory mechanism: {last}")
        self.mem_kind = lib().ft_comm_mem_kind(self._h)
        want_nvls = nvls if nvls is not None else os.environ.get("FT_NVLS", "1") != "0"
        if want_nvls and self.mem_kind == MEM_VMM and world > 1:
            self.has_nvls = self._setup_multicast()
        self._check(lib().ft_comm_finalize(self._h))
        self._configure_from_env()
        log.info(f"communicator up: world {world}, device {dev}, heap {heap_bytes >> 20} MiB + 2 x {staging_bytes >> 20} MiB slots, "
                 f"memory {'vmm' if self.mem_kind == MEM_VMM else 'ipc'}, nvls {'on' if self.has_nvls else 'off'}, "
                 f"shape {'auto' if self.auto else self.default_shape}", rank)
        dist.barrier(group=group)

    def alloc(self, shape, dtype=torch.float32) -> torch.Tensor:
        """As :meth:`_CommBase.alloc`.  With ``FT_CHECK_SYMMETRIC=1`` the call is collective and verifies that
        every rank got the same heap offset and size: in-place collectives read a peer's heap at THIS rank's
        offset, so ranks that allocate in different orders would silently reduce unrelated memory."""
        t = super().alloc(shape, dtype)
        if self._check_symmetric and self.world > 1:
            import torch.distributed as dist
            mine = (t.data_ptr() - (lib().ft_comm_heap_base(self._h) or 0), t.numel() * t.element_size())
            every = [None] * self.world
            dist.all_gather_object(every, mine, group=self.group)
            if any(e != mine for e in every):
                raise FlexTreeError(1, f"asymmetric heap allocation: (offset, bytes) per rank = {every}")
        return t

    # handles travel as pickled bytes (IPC) or as descriptors over unix sockets (VMM)
    def _exchange(self, kind: int) -> bool:
        import torch.distributed as dist
        L, world, rank = lib(), self.world, self.rank
        if world == 1:
            return True
        try:
            if kind == MEM_IPC:
                blob = C.create_string_buffer(64)
                if L.ft_comm_export_ipc(self._h, blob):
                    return False
                blobs = [None] * world
                dist.all_gather_object(blobs, blob.raw, group=self.group)
                for p in range(world):
                    if p != rank and L.ft_comm_import_ipc(self._h, p, C.create_string_buffer(blobs[p], 64)):
                        return False
                return True
            session = [uuid.uuid4().hex if rank == 0 else None]
            dist.broadcast_object_list(session, src=0, group=self.group)
            self._session = session[0]
            sock = L.ft_fd_listen(f"ft-{self._session}-{rank}".encode())
            fd = C.c_int(-1)
            ok = sock >= 0 and L.ft_comm_export_fd(self._h, C.byref(fd)) == 0
            oks = [None] * world
            dist.all_gather_object(oks, bool(ok), group=self.group)   # also: every listener is up
            if not all(oks):
                return False
            for p in range(world):
                if p != rank and L.ft_fd_send(f"ft-{self._session}-{p}".encode(), fd.value, rank, 20000):
                    ok = False
            for _ in range(world - 1):
                tag = C.c_int(-1)
                got = L.ft_fd_recv(sock, C.byref(tag), 20000)
                if got < 0 or L.ft_comm_import_fd(self._h, tag.value, got):
                    ok = False
                if got >= 0:
                    L.ft_fd_close(got)
            L.ft_fd_close(fd.value)
            self._sock = sock
            return ok
        except Exception as e:  # noqa: BLE001 - any bootstrap failure means "try the next mechanism"
            log.warn(f"handle exchange failed: {e}", rank)
            return False

    def _setup_multicast(self) -> bool:
        import torch.distributed as dist
        L, world, rank = lib(), self.world, self.rank

        def agree(flag: bool) -> bool:
            oks = [None] * world
            dist.all_gather_object(oks, bool(flag), group=self.group)
            return all(oks)

        if not agree(bool(L.ft_comm_mc_supported(self._h))):
            return False
        ok = True
        if rank == 0:
            fd = C.c_int(-1)
            ok = L.ft_comm_mc_create(self._h, C.byref(fd)) == 0
            if ok:
                for p in range(1, world):
                    ok = L.ft_fd_send(f"ft-{self._session}-{p}".encode(), fd.value, 1000, 20000) == 0 and ok
                ok = L.ft_comm_mc_join(self._h, -1) == 0 and ok
                L.ft_fd_close(fd.value)
        if not agree(ok):   # rank 0 could not create: nobody waits for a descriptor
            return False
        if rank != 0:
            tag = C.c_int(-1)
            got = L.ft_fd_recv(self._sock, C.byref(tag), 20000)
            ok = got >= 0 and tag.value == 1000 and L.ft_comm_mc_join(self._h, got) == 0
            if got >= 0:
                L.ft_fd_close(got)
        if not agree(ok):   # everyone must have joined before anyone binds
            return False
        ok = L.ft_comm_mc_bind(self._h) == 0
        if not ok:
            log.warn("multicast bind failed: " + L.ft_comm_last_error(self._h).decode(), rank)
        return agree(ok)

    def close(self, collective: bool = True):
        """Collective by default: every rank drains its GPU and meets the others before any memory is
        unmapped, so no peer kernel can still be reading (or multicasting into) a heap that goes away.
        (Garbage collection calls it with collective=False: ranks are not collected in step.)"""
        if self._h and collective:
            try:
                import torch.distributed as dist
                torch.cuda.synchronize(self.device)
                if dist.is_initialized():
                    dist.barrier(group=self.group)
            except Exception as e:  # noqa: BLE001 - e.g. the process group is already gone at interpreter exit
                log.debug(f"close(): no rendezvous before teardown ({e})", self.rank)
        sock = getattr(self, "_sock", -1)
        if sock is not None and sock >= 0:
            lib().ft_fd_close(sock)
            self._sock = -1
        super().close()


class _LocalRank(_CommBase):
    pass


class LocalWorld:
    """All ranks in this process.

    ``devices`` lists one CUDA device per rank.  With distinct devices the ranks' kernels really
    run concurrently and rendezvous over NVLink.  With every rank on the SAME device the world is
    *emulated*: each stage of the plan is launched rank after rank on one stream with the
    rendezvous switched off, so kernels never wait on one another.
    """

    def __init__(self, world: int, devices: Sequence[int] | None = None, heap_bytes: int = 64 << 20,
                 staging_bytes: int = 16 << 20, mem: str = "ipc"):
        devices = list(devices) if devices is not None else [0] * world
        assert len(devices) == world
        self.world = world
        self.emulated = len(set(devices)) < world
        self.ranks: list[_LocalRank] = []
        kind = MEM_VMM if mem == "vmm" else MEM_IPC
        for r in range(world):
            c = _LocalRank()
            with torch.cuda.device(devices[r]):
                code = c._create(r, world, devices[r], heap_bytes, staging_bytes, kind)
            if code:
                raise FlexTreeError(code, lib().ft_comm_last_error(c._h).decode())
            self.ranks.append(c)
        arr = (C.c_void_p * world)(*[c._h for c in self.ranks])
        code = lib().ft_comm_connect_local(arr, world)
        if code:
            raise FlexTreeError(code, lib().ft_comm_last_error(self.ranks[0]._h).decode())
        self._emu_call = 0

    def all_reduce(self, tensors: Sequence[torch.Tensor], op: str = "sum", shape=None, algo: str = "staged",
                   scale: float = 1.0, outs: Sequence[torch.Tensor] | None = None):
        """Rank r reduces ``tensors[r]`` (in place unless ``outs`` is given)."""
        world = self.world
        shp = _as_shape(shape, world) or Shape.flat(world)
        if op == "avg":
            op, scale = "sum", scale / world
        outs = list(outs) if outs is not None else list(tensors)
        if not self.emulated:
            for r, c in enumerate(self.ranks):
                with torch.cuda.device(c.device):
                    c.all_reduce(tensors[r], op=op, shape=shp if algo == "staged" or (algo == "ll" and shape is not None) else None,
                                 algo=algo, scale=scale, out=outs[r])
            return outs
        L = lib()
        dt = ft_dtype(tensors[0].dtype)
        st = C.c_void_p(torch.cuda.current_stream(self.ranks[0].device).cuda_stream)

        def ptrs(r):
            src = None if outs[r].data_ptr() == tensors[r].data_ptr() else tensors[r].data_ptr()
            return src, outs[r].data_ptr()

        if world == 1:
            self.ranks[0].all_reduce(tensors[0], op=op, scale=scale, out=outs[0])
            return outs
        if algo == "push":
            for r, c in enumerate(self.ranks):
                if outs[r].data_ptr() != tensors[r].data_ptr():
                    outs[r].copy_(tensors[r])
            for r, c in enumerate(self.ranks):
                c._check(L.ft_allreduce_emulate_push(c._h, outs[r].data_ptr(), outs[r].numel(), dt, OPS[op], float(scale), st))
            return outs
        if algo == "ll" and shape is not None:
            # a plan on tagged words: per stage every rank pushes, then every rank receives
            nstages = planner.plan_num_stages(world, shp)
            if nstages < 0:
                raise FlexTreeError(4, f"invalid FT_TOPO {shp} ({planner.validate_shape(world, shp)})")
            arr, nw, lonely, ring = shp.c_args()
            for s in range(nstages):
                for phase in (1, 2):
                    for r, c in enumerate(self.ranks):
                        src, dst = ptrs(r)
                        c._check(L.ft_allreduce_emulate_ll_tree(c._h, src, dst, tensors[r].numel(), dt, OPS[op], arr, nw, lonely, ring,
                                                                float(scale), s, phase, self._emu_call, st))
            self._emu_call += 1
            return outs
        if algo == "ll":
            for phase in (1, 2):
                for r, c in enumerate(self.ranks):
                    src, dst = ptrs(r)
                    c._check(L.ft_allreduce_emulate_ll(c._h, src, dst, tensors[r].numel(), dt, OPS[op], float(scale), phase,
                                                       self._emu_call, st))
            self._emu_call += 1
            return outs
        if algo == "oneshot":
            for phase in (1, 4):
                for r, c in enumerate(self.ranks):
                    src, dst = ptrs(r)
                    c._check(L.ft_allreduce_emulate_oneshot(c._h, src, dst, tensors[r].numel(), dt, OPS[op], float(scale),
                                                            phase, self._emu_call, st))
            self._emu_call += 1
            return outs
        nstages = planner.plan_num_stages(world, shp)
        if nstages < 0:
            raise FlexTreeError(4, f"invalid FT_TOPO {shp} ({planner.validate_shape(world, shp)})")
        arr, nw, lonely, ring = shp.c_args()
        # pass -1 publishes every rank's input (the real kernel does this before its opening rendezvous)
        for s in range(-1, nstages):
            for r, c in enumerate(self.ranks):
                src, dst = ptrs(r)
                c._check(L.ft_allreduce_emulate_stage(c._h, src, dst, tensors[r].numel(), dt, OPS[op], arr, nw, lonely, ring,
                                                      float(scale), max(s, 0), s + 1, st))
        return outs

    def _phase(self, tensors: Sequence[torch.Tensor], gather: bool, op: str, shape, scale: float):
        world = self.world
        shp = _as_shape(shape, world) or Shape.flat(world)
        if op == "avg":
            op, scale = "sum", scale / world
        if not self.emulated or world == 1:
            for r, c in enumerate(self.ranks):
                with torch.cuda.device(c.device):
                    if gather:
                        c.all_gather(tensors[r], shape=shp)
                    else:
                        c.reduce_scatter(tensors[r], op=op, shape=shp, scale=scale)
            return shp
        nstages = planner.plan_num_stages(world, shp)
        if nstages < 0:
            raise FlexTreeError(4, f"invalid FT_TOPO {shp} ({planner.validate_shape(world, shp)})")
        arr, nw, lonely, ring = shp.c_args()
        L, dt = lib(), ft_dtype(tensors[0].dtype)
        st = C.c_void_p(torch.cuda.current_stream(self.ranks[0].device).cuda_stream)
        for s in (range(nstages // 2, nstages) if gather else range(nstages // 2)):
            for r, c in enumerate(self.ranks):
                if not c.in_heap(tensors[r]):
                    raise ValueError("reduce_scatter / all_gather work in place on a tensor from alloc()")
                c._check(L.ft_allreduce_emulate_stage(c._h, None, tensors[r].data_ptr(), tensors[r].numel(), dt, OPS[op], arr, nw,
                                                      lonely, ring, float(scale), s, s + 1, st))
        return shp

    def reduce_scatter(self, tensors: Sequence[torch.Tensor], op: str = "sum", shape=None, scale: float = 1.0):
        """Reduce-scatter half alone; returns, per rank, the views of the blocks it holds complete."""
        shp = self._phase(tensors, False, op, shape, scale)
        out = []
        for r, c in enumerate(self.ranks):
            flat = tensors[r].view(-1)
            out.append([flat[slice(*c.block_range(tensors[r], b))] for b in planner.owned_blocks(self.world, shp, r)])
        return out

    def all_gather(self, tensors: Sequence[torch.Tensor], shape=None):
        """All-gather half alone, in place."""
        self._phase(tensors, True, "sum", shape, 1.0)
        return tensors

    def profile_stages(self, tensors: Sequence[torch.Tensor], shape, op: str = "sum", iters: int = 5) -> list[float]:
        """Per-stage device time (ms, all ranks of the stage together) of a staged plan on an emulated
        world: CUDA events around each stage's launches.  The counterpart of the reference's SHOW_TIME
        phase log (allreduce_over_mpi/mpi_mod.hpp:31-35), which times its two phases on the host."""
        if not self.emulated:
            raise RuntimeError("per-stage timing needs the single-GPU emulated world")
        shp = _as_shape(shape, self.world) or Shape.flat(self.world)
        nstages = planner.plan_num_stages(self.world, shp)
        arr, nw, lonely, ring = shp.c_args()
        L, dt = lib(), ft_dtype(tensors[0].dtype)
        st = C.c_void_p(torch.cuda.current_stream(self.ranks[0].device).cuda_stream)
        acc = [0.0] * (nstages + 1)
        for _ in range(iters):
            for s in range(-1, nstages):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for r, c in enumerate(self.ranks):
                    c._check(L.ft_allreduce_emulate_stage(c._h, None, tensors[r].data_ptr(), tensors[r].numel(), dt, OPS[op], arr, nw,
                                                          lonely, ring, 1.0, max(s, 0), s + 1, st))
                b.record()
                b.synchronize()
                acc[s + 1] += a.elapsed_time(b) / iters
        return acc   # [publish, stage 0, stage 1, ...]

    def close(self):
        for c in self.ranks:
            c.close()
        self.ranks = []
