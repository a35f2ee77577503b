"""Python face of the MPI_Allreduce-compatible entry point (csrc/api/flextree_mpi.h).

    world = ThreadWorld(6)                      # ranks are threads, host buffers
    comm = world.comm(rank)
    MPI_Allreduce_FT(IN_PLACE, tensor, tensor.numel(), MPI_FLOAT, MPI_SUM, comm)

    comm = from_flextree_comm(FlexTreeComm(...))   # GPU ranks; device or host tensors

The tree shape comes from the environment (FT_TOPO / FT_LONELY), read on every call, exactly
like the reference's entry point (allreduce_over_mpi/mpi_mod.hpp:1723-1778, :1419-1486).
Return value 0 means success; failures return the ft_status code after printing the
reference's message ("Type ... is not supported in MPI mode.", "Unsupported op ...",
"invalid FT_TOPO ...") instead of exiting the process.
"""
from __future__ import annotations

import ctypes as C

import torch

from .._lib import DTYPES, lib

IN_PLACE = C.c_void_p(1)
MPI_IN_PLACE = IN_PLACE
MPI_UINT8_T, MPI_INT8_T = DTYPES["uint8"], DTYPES["int8"]
MPI_UINT16_T, MPI_INT16_T = DTYPES["uint16"], DTYPES["int16"]
MPI_INT32_T, MPI_INT64_T = DTYPES["int32"], DTYPES["int64"]
MPI_FLOAT, MPI_DOUBLE, MPI_C_BOOL = DTYPES["float32"], DTYPES["float64"], DTYPES["bool"]
MPI_LONG_LONG = MPI_LONG_LONG_INT = DTYPES["int64"]
FT_UINT32_T, FT_UINT64_T, FT_BFLOAT16, FT_FLOAT16 = DTYPES["uint32"], DTYPES["uint64"], DTYPES["bfloat16"], DTYPES["float16"]
MPI_SUM, MPI_BAND = 0, 1
MPI_MAX = 100   # stands for "any operator FlexTree does not implement"


def _ptr(buf):
    if buf is None:
        return None
    if isinstance(buf, C.c_void_p):
        return buf
    if isinstance(buf, torch.Tensor):
        return C.c_void_p(buf.data_ptr())
    return C.c_void_p(int(buf))


class Comm:
    def __init__(self, handle, keep=None):
        self._h = C.c_void_p(handle)
        self._keep = keep

    def size(self) -> int:
        n = C.c_int()
        lib().FT_Comm_size(self._h, C.byref(n))
        return n.value

    def rank(self) -> int:
        n = C.c_int()
        lib().FT_Comm_rank(self._h, C.byref(n))
        return n.value

    def free(self):
        if self._h:
            lib().ft_mpi_comm_free(self._h)
            self._h = C.c_void_p()


class ThreadWorld:
    """Ranks are threads of this process (each thread calls MPI_Allreduce_FT with its own comm)."""

    def __init__(self, world: int, timeout_s: float = 10.0):
        self.world = world
        self._w = lib().ft_cpu_world_create(world, timeout_s)

    def comm(self, rank: int) -> Comm:
        return Comm(lib().ft_mpi_thread_rank(self._w, rank), keep=self)

    def close(self):
        if self._w:
            lib().ft_cpu_world_destroy(self._w)
            self._w = None


def from_flextree_comm(comm, stream=None) -> Comm:
    """MPI-style communicator over a GPU :class:`FlexTreeComm` (collectives run on ``stream``)."""
    st = stream.cuda_stream if stream is not None else torch.cuda.current_stream(comm.device).cuda_stream
    return Comm(lib().ft_mpi_from_comm(comm._h, C.c_void_p(st)), keep=comm)


def MPI_Allreduce_FT(sendbuf, recvbuf, count: int, datatype: int, op: int, comm: Comm) -> int:
    return lib().MPI_Allreduce_FT_c(_ptr(sendbuf), _ptr(recvbuf), count, datatype, op, comm._h)


def last_error() -> str:
    return lib().ft_mpi_last_error().decode()
