"""Descriptor passing between processes (the bootstrap of VMM handle exchange), on CPU."""
import ctypes as C
import multiprocessing as mp
import os

from allreduce_over_mpi_b200 import lib


def _child(name, tag):
    L = lib()
    r, w = os.pipe()
    os.write(w, f"from-{tag}".encode())
    assert L.ft_fd_send(name.encode(), r, tag, 5000) == 0


def test_two_senders_one_listener():
    L = lib()
    name = f"ft-test-{os.getpid()}"
    s = L.ft_fd_listen(name.encode())
    assert s >= 0
    ctx = mp.get_context("spawn")   # fork in a process that already runs OpenMP threads can deadlock the child
    ps = [ctx.Process(target=_child, args=(name, t)) for t in (3, 7)]
    [p.start() for p in ps]
    got = {}
    for _ in ps:
        tag = C.c_int(-1)
        fd = L.ft_fd_recv(s, C.byref(tag), 5000)
        assert fd >= 0
        got[tag.value] = os.read(fd, 32).decode()
        os.close(fd)
    [p.join() for p in ps]
    assert got == {3: "from-3", 7: "from-7"}
    L.ft_fd_close(s)


def test_timeouts_instead_of_blocking():
    L = lib()
    s = L.ft_fd_listen(f"ft-test-idle-{os.getpid()}".encode())
    tag = C.c_int(-1)
    assert L.ft_fd_recv(s, C.byref(tag), 50) == -1          # nobody sends
    assert L.ft_fd_send(b"ft-test-nobody-listens", 0, 1, 50) == -2
    L.ft_fd_close(s)
