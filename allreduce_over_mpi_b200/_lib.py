"""ctypes loader for libflextree.so.

The library is built in-tree by :mod:`allreduce_over_mpi_b200.build`.  If it is missing the
import fails loudly: there is no pure-Python fallback for the kernels.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libflextree.so"

FT_MAX_FANIN = 32
FT_MAX_RANKS = 64

# ft_dtype / ft_op / ft_status mirror csrc/api/ft_types.h
DTYPES = {"uint8": 0, "int8": 1, "uint16": 2, "int16": 3, "int32": 4, "int64": 5, "float32": 6,
          "float64": 7, "bool": 8, "uint32": 9, "uint64": 10, "bfloat16": 11, "float16": 12}
DTYPE_SIZE = {0: 1, 1: 1, 2: 2, 3: 2, 4: 4, 5: 8, 6: 4, 7: 8, 8: 1, 9: 4, 10: 8, 11: 2, 12: 2}
OPS = {"sum": 0, "band": 1}
STATUS = {0: "ok", 1: "invalid argument", 2: "unsupported type", 3: "unsupported op", 4: "invalid topology",
          5: "timeout waiting for a peer", 6: "CUDA error", 7: "size exceeds limit", 8: "protocol error",
          9: "not available", 10: "address outside the symmetric heap (access skipped)"}


class FlexTreeError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        self.code = code
        super().__init__(f"flextree: {STATUS.get(code, code)}{': ' + what if what else ''}")


class V1Params(C.Structure):
    _fields_ = [("launch_us", C.c_double), ("sync_us", C.c_double), ("link_gbs", C.c_double),
                ("hbm_gbs", C.c_double), ("stage_floor_us", C.c_double), ("nvls_gbs", C.c_double),
                ("oneshot_max_bytes", C.c_double), ("ll_us", C.c_double), ("ll_max_bytes", C.c_double),
                ("push_gain", C.c_double), ("peer_eff", C.c_double * (FT_MAX_RANKS + 1))]


class Choice(C.Structure):
    """ft_choice of csrc/api/flextree.h: what the selection policy picked for a message."""
    _fields_ = [("algo", C.c_int), ("nw", C.c_int), ("widths", C.c_int * 16), ("lonely", C.c_int), ("ring", C.c_int),
                ("from_table", C.c_int), ("hybrid_bytes", C.c_double), ("hybrid_lanes", C.c_double),
                ("algo_name", C.c_char * 16)]


_lib = None


def _declare(lib):
    i, u64, sz, dbl, vp, cp = C.c_int, C.c_uint64, C.c_size_t, C.c_double, C.c_void_p, C.c_char_p
    ip = C.POINTER(C.c_int)
    shape = [ip, i, i, i]  # widths, nw, lonely, ring
    sig = {
        "ft_version": (cp, []),
        "ft_prime_factors": (i, [i, ip, i]),
        "ft_is_prime": (i, [i]),
        "ft_is_prime_loose": (i, [i]),
        "ft_count_ordered_factorizations": (u64, [i]),
        "ft_candidate_shapes": (sz, [i, i, cp, sz]),
        "ft_choose_width": (sz, [i, cp, sz]),
        "ft_cost_v0": (dbl, [ip, i, i, dbl]),
        "ft_choose_v0": (i, [i, dbl, ip, i, C.POINTER(dbl), C.POINTER(u64)]),
        "ft_v1_defaults": (None, [C.POINTER(V1Params)]),
        "ft_cost_v1": (dbl, [i, *shape, u64, C.POINTER(V1Params)]),
        "ft_cost_v1_oneshot": (dbl, [i, u64, C.POINTER(V1Params)]),
        "ft_cost_v1_nvls": (dbl, [i, u64, C.POINTER(V1Params)]),
        "ft_pick_algorithm": (i, [i, u64, C.POINTER(V1Params), i, i, ip, i, ip, ip, cp, sz, C.POINTER(dbl)]),
        "ft_pick_algorithm2": (i, [i, u64, C.POINTER(V1Params), i, i, i, ip, i, ip, ip, cp, sz, C.POINTER(dbl)]),
        "ft_executable_shapes": (sz, [i, cp, sz]),
        "ft_policy_create": (vp, [i]),
        "ft_policy_destroy": (None, [vp]),
        "ft_policy_default_path": (sz, [cp, sz]),
        "ft_policy_load": (i, [vp, cp, cp, sz]),
        "ft_policy_set_params": (i, [vp, C.POINTER(V1Params)]),
        "ft_policy_get_params": (i, [vp, C.POINTER(V1Params)]),
        "ft_policy_clear_rows": (None, [vp]),
        "ft_policy_num_rows": (i, [vp]),
        "ft_policy_add_row": (i, [vp, u64, cp, cp]),
        "ft_policy_choose": (i, [vp, u64, i, i, u64, u64, i, C.POINTER(Choice)]),
        "ft_parse_topo": (i, [cp, cp, i, ip, i, ip, ip, ip, ip, cp, sz]),
        "ft_validate_shape": (i, [i, *shape, cp, sz]),
        "ft_plan_check": (i, [i, *shape, cp, sz]),
        "ft_plan_num_stages": (i, [i, *shape]),
        "ft_plan_max_fanin": (i, [i, *shape]),
        "ft_plan_traffic": (u64, [i, *shape, u64, u64]),
        "ft_plan_describe": (sz, [i, *shape, i, u64, u64, cp, sz]),
        "ft_plan_json": (sz, [i, *shape, cp, sz]),
        "ft_cpu_reduce": (i, [i, i, C.POINTER(vp), vp, i, sz, i]),
        "ft_run_plan_snapshot": (i, [i, *shape, i, i, C.POINTER(vp), u64, u64]),
        "ft_run_plan_snapshot_range": (i, [i, *shape, i, i, C.POINTER(vp), u64, u64, i, i]),
        "ft_plan_rs_holders": (i, [i, *shape, C.POINTER(u64)]),
        "ft_dev_plan_check": (i, [i, *shape, i, C.c_char_p, sz]),
        "ft_context_describe": (sz, [i, i, i, u64, i, C.c_char_p, sz]),
        "ft_cpu_world_create": (vp, [i, dbl]),
        "ft_cpu_world_destroy": (None, [vp]),
        "ft_cpu_allreduce": (i, [vp, i, *shape, i, i, vp, vp, u64, u64, i, i, i, ip]),
        "ft_cpu_phase": (i, [vp, i, *shape, i, i, vp, u64, u64, i, ip]),
        "ft_proc_world_join": (vp, [C.c_char_p, i, i, C.c_double, C.c_char_p, sz]),
        "ft_proc_world_leave": (None, [vp]),
        "ft_proc_world_rank": (i, [vp]),
        "ft_proc_world_size": (i, [vp]),
        "ft_proc_barrier": (i, [vp]),
        "ft_proc_last_error": (C.c_char_p, [vp]),
        "ft_proc_allreduce": (i, [vp, *shape, i, i, vp, vp, u64, ip]),
        "ft_proc_phase": (i, [vp, *shape, i, i, vp, u64, i, ip]),
        "ft_proc_heap_create": (i, [vp, sz]),
        "ft_proc_alloc": (vp, [vp, sz]),
        "ft_proc_free": (i, [vp, vp]),
        "ft_proc_heap_symmetric": (i, [vp, vp]),
        "ft_mpi_thread_rank": (vp, [vp, i]),
        "ft_mpi_from_comm": (vp, [vp, vp]),
        "ft_mpi_comm_free": (None, [vp]),
        "FT_Comm_size": (i, [vp, ip]),
        "FT_Comm_rank": (i, [vp, ip]),
        "FT_Type_size": (i, [i, ip]),
        "FT_Type_get_name": (i, [i, cp, ip]),
        "MPI_Allreduce_FT": (i, [vp, vp, i, i, i, vp]),
        "MPI_Allreduce_FT_c": (i, [vp, vp, sz, i, i, vp]),
        "FT_enabled": (None, []),
        "ft_mpi_last_error": (cp, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def lib() -> C.CDLL:
    """The loaded library (built on first use when nvcc is available)."""
    global _lib
    if _lib is None:
        path = LIB_PATH
        if os.environ.get("FT_LIB", "") == "bounds":   # the debugging build whose kernels range-check every heap access
            path = LIB_PATH.with_name("libflextree_bounds.so")
            if not path.exists():
                from .build import build_bounds
                path = build_bounds()
        elif not path.exists() or os.environ.get("FT_REBUILD"):
            from .build import ensure_built
            path = ensure_built()
        if not path.exists():
            raise ImportError(f"{path} is missing; run `python -m allreduce_over_mpi_b200.build`")
        _lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        _declare(_lib)
        from . import _lib_cuda
        _lib_cuda.declare(_lib)
    return _lib


def text_call(fn, *args, cap: int = 1 << 16) -> str:
    """Call an API function whose last two parameters are (buf, cap) and return the string."""
    while True:
        buf = C.create_string_buffer(cap)
        need = fn(*args, buf, cap)
        if need < cap:
            return buf.value.decode()
        cap = need + 1


def check(code: int, what: str = "") -> None:
    if code != 0:
        raise FlexTreeError(code, what)
