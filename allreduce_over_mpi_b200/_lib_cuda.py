"""ctypes signatures of the CUDA half of libflextree.so (kernels + communicator)."""
from __future__ import annotations

import ctypes as C


def declare(lib) -> None:
    i, u64, sz, vp, cp, f32 = C.c_int, C.c_uint64, C.c_size_t, C.c_void_p, C.c_char_p, C.c_float
    sig = {
        "ft_reduce_nway": (i, [i, i, C.POINTER(vp), vp, i, sz, i, vp]),
        "ft_reduce_nway_scaled": (i, [i, i, C.POINTER(vp), vp, i, sz, f32, vp]),
        "ft_last_cuda_error": (cp, []),
        "ft_launch_count": (u64, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise ImportError(f"libflextree.so lacks {name}; rebuild with python -m allreduce_over_mpi_b200.build")
        fn.restype = res
        fn.argtypes = args
