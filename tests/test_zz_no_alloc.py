"""The allocation-free all-reduce entry point, called through its exported C symbol.

Some users of the library may not allocate device memory at the moment they need a reduction
(a plug-in inside a host application that owns all GPU memory, a loop that cannot afford
cudaMalloc's implicit synchronisation, a point of the program where the runtime accepts no
allocation call).  ft_local_allreduce_noalloc() serves them from a fixed
8 MiB array inside the library.  Here its result is compared with the regular path (a one-shot
all-reduce through communicators, which allocate heaps) on two calls in a row: the second call
runs over whatever the first one left in the shared array.

Collected last on purpose (file name), so a run that stops at the first failure has already run
everything else.  Works alone in a fresh process and after the other tests.
"""
import ctypes as C

import pytest
import torch

from allreduce_over_mpi_b200._lib import DTYPES, LIB_PATH, OPS
from allreduce_over_mpi_b200.parallel.comm import LocalWorld

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH = 8 << 20


def entry():
    lib = C.CDLL(str(LIB_PATH))          # plain dlopen of the shipped library: the C symbol is the interface under test
    fn = lib.ft_local_allreduce_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_float, C.c_void_p]
    lib.ft_noalloc_last_error.restype = C.c_char_p
    return lib, fn


def call(fn, bufs, dtype_name, op="sum", scale=1.0):
    arr = (C.c_void_p * len(bufs))(*[b.data_ptr() for b in bufs])
    st = torch.cuda.current_stream().cuda_stream
    return fn(arr, len(bufs), bufs[0].numel(), DTYPES[dtype_name], OPS[op], scale, C.c_void_p(st))


def make(n, count, dtype, seed):
    out = []
    for r in range(n):
        g = torch.Generator().manual_seed(seed * 100 + r)
        x = torch.rand(count, generator=g, dtype=torch.float64) * 2 - 1
        out.append((x.to(dtype) if dtype.is_floating_point else (x * 50).to(dtype)).to(DEV))
    return out


@pytest.mark.parametrize("dtype,name,tol", [(torch.float32, "float32", 1e-5), (torch.bfloat16, "bfloat16", 0.15)])
def test_matches_the_allocating_path_twice_in_a_row(dtype, name, tol):
    lib, fn = entry()
    n = 4
    world = LocalWorld(n, heap_bytes=1 << 20, staging_bytes=4 << 20)
    # two different problems back to back: the second one finds the first one's data in the array
    for rnd, count in enumerate((100_003, 37_777)):
        a = make(n, count, dtype, seed=rnd)
        b = [t.clone() for t in a]
        want = torch.stack([t.double() for t in a]).sum(0)
        assert call(fn, a, name) == 0, lib.ft_noalloc_last_error()
        world.all_reduce(b, algo="oneshot")
        torch.cuda.synchronize()
        for r in range(n):
            assert torch.allclose(a[r].double(), b[r].double(), atol=tol, rtol=0), (rnd, r)
            assert torch.allclose(a[r].double(), want, atol=tol * 2, rtol=0), (rnd, r)
    world.close()


def test_scale_band_and_limits():
    lib, fn = entry()
    x = make(3, 5000, torch.float32, seed=7)
    want = torch.stack(x).sum(0) / 3
    assert call(fn, x, "float32", scale=1 / 3) == 0
    torch.cuda.synchronize()
    assert all(torch.allclose(t, want, atol=1e-6) for t in x)
    m = [torch.full((999,), 0xFF ^ (1 << r), dtype=torch.int32, device=DEV) for r in range(4)]
    assert call(fn, m, "int32", op="band") == 0
    torch.cuda.synchronize()
    assert all(bool((t == 0xF0).all()) for t in m)
    # beyond the built-in staging area: refused with a message, nothing launched, inputs untouched
    big = [torch.ones((SCRATCH // 4 // 2) + 1024, device=DEV) for _ in range(2)]
    assert call(fn, big, "float32") == 7
    assert b"built-in area holds 8388608" in lib.ft_noalloc_last_error()
    torch.cuda.synchronize()
    assert bool((big[0] == 1).all())
    # exactly at the limit is accepted
    fit = [torch.ones(SCRATCH // 4 // 2, device=DEV) for _ in range(2)]
    assert call(fn, fit, "float32") == 0
    torch.cuda.synchronize()
    assert bool((fit[1] == 2).all())
    assert call(fn, [torch.ones(4, device=DEV)], "float32", op="band") == 2     # float AND: unsupported type


def test_buffers_off_the_16_byte_grid_take_the_element_wise_path():
    """Buffers that start one element past a 16-byte boundary (views into larger tensors): the kernels fall back
    to element-sized accesses at both ends and give the same sums as the allocating path, twice in a row."""
    lib, fn = entry()
    n = 3
    world = LocalWorld(n, heap_bytes=1 << 20, staging_bytes=1 << 20)
    for rnd, (dtype, name, tol) in enumerate(((torch.float32, "float32", 1e-5), (torch.bfloat16, "bfloat16", 0.15))):
        whole = make(n, 20_011, dtype, seed=20 + rnd)
        a = [t[1:] for t in whole]                 # data_ptr is 4 (or 2) bytes past the allocation's 256-byte boundary
        assert all(t.data_ptr() % 16 != 0 for t in a)
        b = [t.clone() for t in a]
        heads = [t[0].item() for t in whole]
        assert call(fn, a, name) == 0, lib.ft_noalloc_last_error()
        world.all_reduce(b, algo="oneshot")
        torch.cuda.synchronize()
        for r in range(n):
            assert torch.allclose(a[r].double(), b[r].double(), atol=tol, rtol=0), (name, r)
            assert whole[r][0].item() == heads[r]                 # the element before the view is untouched
    world.close()
