"""ctypes signatures of the CUDA half of libflextree.so (kernels + communicator)."""
from __future__ import annotations

import ctypes as C


def declare(lib) -> None:
    i, u64, sz, vp, cp, f32, dbl = C.c_int, C.c_uint64, C.c_size_t, C.c_void_p, C.c_char_p, C.c_float, C.c_double
    ip = C.POINTER(C.c_int)
    shape = [ip, i, i, i]
    sig = {
        "ft_reduce_nway": (i, [i, i, C.POINTER(vp), vp, i, sz, i, vp]),
        "ft_reduce_nway_scaled": (i, [i, i, C.POINTER(vp), vp, i, sz, f32, vp]),
        "ft_scale_inplace": (i, [i, vp, sz, f32, vp]),
        "ft_last_cuda_error": (cp, []),
        "ft_launch_count": (u64, []),
        "ft_host_pipe_create": (i, [i, sz, i, i, C.POINTER(vp)]),
        "ft_host_pipe_destroy": (None, [vp]),
        "ft_host_pipe_last_error": (cp, [vp]),
        "ft_host_pipe_reduce": (i, [vp, i, i, C.POINTER(vp), i, ip, C.POINTER(vp), i, sz, vp]),
        "ft_allreduce_host": (i, [vp, vp, vp, sz, i, i, *shape, i, f32, vp]),
        "ft_comm_set_host_chunk": (None, [vp, sz]),
        "ft_comm_create": (i, [i, i, i, sz, sz, i, C.POINTER(vp)]),
        "ft_comm_destroy": (i, [vp]),
        "ft_comm_last_error": (cp, [vp]),
        "ft_comm_export_fd": (i, [vp, ip]),
        "ft_comm_import_fd": (i, [vp, i, i]),
        "ft_comm_export_ipc": (i, [vp, vp]),
        "ft_comm_import_ipc": (i, [vp, i, vp]),
        "ft_comm_connect_local": (i, [C.POINTER(vp), i]),
        "ft_comm_finalize": (i, [vp]),
        "ft_comm_mc_supported": (i, [vp]),
        "ft_comm_mc_create": (i, [vp, ip]),
        "ft_comm_mc_join": (i, [vp, i]),
        "ft_comm_mc_bind": (i, [vp]),
        "ft_comm_has_nvls": (i, [vp]),
        "ft_comm_heap_base": (vp, [vp]),
        "ft_comm_heap_bytes": (sz, [vp]),
        "ft_comm_alloc": (vp, [vp, sz]),
        "ft_comm_alloc_reset": (None, [vp]),
        "ft_comm_free": (i, [vp, vp]),
        "ft_comm_heap_free_bytes": (sz, [vp]),
        "ft_comm_rank": (i, [vp]),
        "ft_comm_world": (i, [vp]),
        "ft_comm_mem_kind": (i, [vp]),
        "ft_comm_set_timeout_ms": (None, [vp, dbl]),
        "ft_comm_set_max_lanes": (None, [vp, i]),
        "ft_comm_set_oneshot_max": (None, [vp, sz]),
        "ft_comm_set_hybrid": (None, [vp, dbl, dbl]),
        "ft_comm_set_ll_max": (None, [vp, sz]),
        "ft_comm_set_nvls_ctas_per_sm": (None, [vp, i]),
        "ft_comm_set_nvls_config": (i, [vp, i, i, i, i, sz]),
        "ft_comm_set_phase_nvls": (None, [vp, i]),
        "ft_comm_set_nvls1_max_lanes": (None, [vp, i]),
        "ft_bounds_build": (i, []),
        "ft_bounds_check_host": (i, [u64, i, i, u64, u64]),
        "ft_comm_policy": (vp, [vp]),
        "ft_comm_choose": (i, [vp, sz, i, i, vp, vp]),
        "ft_allreduce_emulate_push": (i, [vp, vp, sz, i, i, f32, vp]),
        "ft_allreduce_emulate_ll": (i, [vp, vp, vp, sz, i, i, f32, i, u64, vp]),
        "ft_allreduce_emulate_ll_tree": (i, [vp, vp, vp, sz, i, i, *shape, f32, i, i, u64, vp]),
        "ft_comm_set_ll_tree_max": (None, [vp, sz]),
        "ft_allreduce": (i, [vp, vp, vp, sz, i, i, *shape, i, f32, vp]),
        "ft_reduce_scatter": (i, [vp, vp, sz, i, i, *shape, f32, vp]),
        "ft_all_gather": (i, [vp, vp, sz, i, *shape, vp]),
        "ft_comm_block_elems": (u64, [vp, sz, i]),
        "ft_block_elems": (u64, [u64, i, i]),
        "ft_allreduce_emulate_stage": (i, [vp, vp, vp, sz, i, i, *shape, f32, i, i, vp]),
        "ft_allreduce_emulate_oneshot": (i, [vp, vp, vp, sz, i, i, f32, i, u64, vp]),
        "ft_comm_status": (i, [vp, ip]),
        "ft_comm_stats": (i, [vp, C.POINTER(u64), C.POINTER(u64)]),
        "ft_comm_clear_status": (None, [vp]),
        "ft_comm_wait_probe": (i, [vp, i, dbl, vp]),
        "ft_fd_listen": (i, [cp]),
        "ft_fd_send": (i, [cp, i, i, i]),
        "ft_fd_recv": (i, [i, ip, i]),
        "ft_fd_close": (None, [i]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise ImportError(f"libflextree.so lacks {name}; rebuild with python -m allreduce_over_mpi_b200.build")
        fn.restype = res
        fn.argtypes = args
