"""n-way element-wise reduction: ``out = t[0] (op) t[1] (op) ... (op) t[n-1]``.

CUDA tensors run the sm_100a kernels of ``csrc/kernels/reduce_nway.cu``; CPU tensors run
the host kernels of ``csrc/planner/cpu_reduce.hpp`` (the oracle and the CPU baseline).
Counterpart of the reference's ``reduce_sum_gpu<T>`` launcher
(vector_add/reduce_sum_gpu.h:205-316) and CPU ``reduce_sum`` / ``reduce_band``
(allreduce_over_mpi/mpi_mod.hpp:812-1251).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from .._lib import DTYPES, FT_MAX_FANIN, OPS, check, lib

_TORCH2FT = {
    torch.uint8: "uint8", torch.int8: "int8", torch.int16: "int16", torch.int32: "int32",
    torch.int64: "int64", torch.float32: "float32", torch.float64: "float64", torch.bool: "bool",
    torch.bfloat16: "bfloat16", torch.float16: "float16",
}
for _name in ("uint16", "uint32", "uint64"):
    if hasattr(torch, _name):
        _TORCH2FT[getattr(torch, _name)] = _name


def ft_dtype(dtype: torch.dtype) -> int:
    try:
        return DTYPES[_TORCH2FT[dtype]]
    except KeyError:
        raise TypeError(f"Type {dtype} is not supported") from None


def _ptr_array(tensors: Sequence[torch.Tensor]):
    arr = (C.c_void_p * len(tensors))()
    for k, t in enumerate(tensors):
        arr[k] = t.data_ptr()
    return arr


def _check_inputs(tensors, out):
    if not 1 <= len(tensors) <= FT_MAX_FANIN:
        raise ValueError(f"need 1..{FT_MAX_FANIN} inputs, got {len(tensors)}")
    t0 = tensors[0]
    for t in tensors:
        if t.dtype != t0.dtype or t.numel() != t0.numel() or t.device != t0.device:
            raise ValueError("inputs must share dtype, size and device")
        if not t.is_contiguous():
            raise ValueError("inputs must be contiguous")
    if out is not None and (not out.is_contiguous() or out.numel() != t0.numel() or out.device != t0.device):
        raise ValueError("out must be contiguous, same size and device")


def reduce_nway(tensors: Sequence[torch.Tensor], op: str = "sum", out: torch.Tensor | None = None,
                variant: int = 0, threads: int = 0) -> torch.Tensor:
    """Reduce ``tensors`` element-wise into ``out`` (allocated when omitted).

    ``variant`` selects the device data path: 0/1 vector loads, 2 TMA bulk pipeline,
    11..16 tuning configurations of the vector path (fp32 / bf16 only).
    """
    _check_inputs(tensors, out)
    t0 = tensors[0]
    if out is None:
        out = torch.empty_like(t0)
    elif out.dtype != t0.dtype:
        raise ValueError("out dtype must match inputs (use reduce_nway_scaled to cast)")
    srcs = _ptr_array(tensors)
    dt = ft_dtype(t0.dtype)
    if t0.is_cuda:
        with torch.cuda.device(t0.device):
            stream = torch.cuda.current_stream().cuda_stream
            code = lib().ft_reduce_nway(OPS[op], dt, srcs, out.data_ptr(), len(tensors), t0.numel(), variant,
                                        C.c_void_p(stream))
        check(code, lib().ft_last_cuda_error().decode() if code == 6 else f"{op} on {t0.dtype}")
    else:
        check(lib().ft_cpu_reduce(OPS[op], dt, srcs, out.data_ptr(), len(tensors), t0.numel(), threads),
              f"{op} on {t0.dtype}")
    return out


def cpu_reduce(tensors: Sequence[torch.Tensor], op: str = "sum", threads: int = 0) -> torch.Tensor:
    """Host n-way reduce of CPU tensors (multi-threaded with OpenMP)."""
    return reduce_nway([t.cpu() for t in tensors], op=op, threads=threads)


def reduce_nway_scaled(tensors: Sequence[torch.Tensor], scale: float = 1.0,
                       out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = scale * sum(tensors)`` with fp32 accumulation and an optional fp32<->bf16 cast
    fused into the store (gradient averaging: scale = 1/world, bf16 out)."""
    _check_inputs(tensors, out)
    t0 = tensors[0]
    if not t0.is_cuda:
        raise ValueError("reduce_nway_scaled is a device kernel")
    out_dtype = out_dtype or (out.dtype if out is not None else t0.dtype)
    if out is None:
        out = torch.empty(t0.shape, dtype=out_dtype, device=t0.device)
    with torch.cuda.device(t0.device):
        stream = torch.cuda.current_stream().cuda_stream
        code = lib().ft_reduce_nway_scaled(ft_dtype(t0.dtype), ft_dtype(out.dtype), _ptr_array(tensors),
                                           out.data_ptr(), len(tensors), t0.numel(), float(scale), C.c_void_p(stream))
    check(code, lib().ft_last_cuda_error().decode() if code == 6 else f"{t0.dtype}->{out.dtype}")
    return out


def launch_count() -> int:
    """Kernels launched by libflextree in this process so far."""
    return int(lib().ft_launch_count())


class HostReducePipeline:
    """n-way reductions of vectors that live in pinned HOST memory, streamed through one GPU.

    ``run(inputs, fanins, outs)`` computes ``outs[j] = inputs[0] (op) ... (op) inputs[fanins[j]-1]`` for every j.
    The vectors are cut into chunks; the host-to-device copy of chunk k+1, the reductions of chunk k and the
    device-to-host copy of chunk k-1 run at the same time on three streams (native: csrc/runtime/host_pipeline.cpp),
    so a call costs about max(bytes in, bytes out) over the PCIe rate, where copy in / kernel / copy out one after
    the other (what the reference's benchmark does, vector_add/vector_add.cu:81-136) costs their sum.
    """

    def __init__(self, device=None, chunk_bytes: int = 16 << 20, max_inputs: int = 8, max_outputs: int = 4):
        dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.device = dev
        self._h = C.c_void_p()
        with torch.cuda.device(dev):
            code = lib().ft_host_pipe_create(dev.index or 0, chunk_bytes, max_inputs, max_outputs, C.byref(self._h))
        if code:
            what = lib().ft_host_pipe_last_error(self._h).decode() if self._h else ""
            self.close()
            check(code, what)

    def run(self, inputs: Sequence[torch.Tensor], fanins: Sequence[int], outs: Sequence[torch.Tensor], op: str = "sum",
            stream: torch.cuda.Stream | None = None) -> Sequence[torch.Tensor]:
        """Asynchronous for pinned tensors: the results are complete once ``stream`` (default: the current
        stream of the pipeline's device) has been synchronised."""
        t0 = inputs[0]
        for t in list(inputs) + list(outs):
            if t.is_cuda or not t.is_contiguous() or t.dtype != t0.dtype or t.numel() != t0.numel():
                raise ValueError("inputs and outputs must be contiguous CPU tensors of one dtype and size")
        if len(fanins) != len(outs):
            raise ValueError("one fan-in per output")
        fan = (C.c_int * len(fanins))(*[int(f) for f in fanins])
        with torch.cuda.device(self.device):
            st = (stream or torch.cuda.current_stream()).cuda_stream
            code = lib().ft_host_pipe_reduce(self._h, OPS[op], ft_dtype(t0.dtype), _ptr_array(inputs), len(inputs), fan,
                                             _ptr_array(outs), len(outs), t0.numel(), C.c_void_p(st))
        check(code, lib().ft_host_pipe_last_error(self._h).decode() if code else "")
        return outs

    def close(self):
        if self._h:
            lib().ft_host_pipe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter teardown
            pass
