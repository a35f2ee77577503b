"""MPI_Allreduce-compatible entry point with ranks as threads (host buffers): the benchmark
configuration of the reference - N = 6 with FT_TOPO=2,3 and N = 7 with FT_TOPO=2,3 FT_LONELY=1,
1 048 576 floats per rank, uniform[-1,1) seeded by rank, checked against an fp64 sum."""
import os
import threading

import pytest
import torch

from allreduce_over_mpi_b200.parallel import mpi_compat as M


def run_world(world, fn):
    tw = M.ThreadWorld(world, timeout_s=20)
    out = [None] * world

    def work(r):
        comm = tw.comm(r)
        out[r] = fn(r, comm)
        comm.free()

    ts = [threading.Thread(target=work, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    tw.close()
    return out


def make(rank, n=1_048_576, dtype=torch.float32):
    g = torch.Generator().manual_seed(rank)
    return (torch.rand(n, generator=g, dtype=torch.float64) * 2 - 1).to(dtype)


@pytest.fixture
def env():
    saved = {k: os.environ.get(k) for k in ("FT_TOPO", "FT_LONELY")}
    yield os.environ
    for k, v in saved.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


@pytest.mark.parametrize("world,topo,lonely", [(6, "2,3", None), (7, "2,3", "1"), (6, None, None), (5, "1", None),
                                               (8, "2,2,2", None), (6, "2,2", "2"), (4, "auto", None)])
def test_reference_benchmark_configs(env, world, topo, lonely):
    env.pop("FT_TOPO", None); env.pop("FT_LONELY", None)
    if topo:
        env["FT_TOPO"] = topo
    if lonely:
        env["FT_LONELY"] = lonely
    n = 1_048_576 if world <= 7 else 100_003
    want = torch.stack([make(r, n).double() for r in range(world)]).sum(0)

    def rank_fn(r, comm):
        assert comm.size() == world and comm.rank() == r
        data = make(r, n)
        rc = M.MPI_Allreduce_FT(M.IN_PLACE, data, n, M.MPI_FLOAT, M.MPI_SUM, comm)
        # out of place as well
        src, dst = make(r, n), torch.zeros(n)
        rc2 = M.MPI_Allreduce_FT(src, dst, n, M.MPI_FLOAT, M.MPI_SUM, comm)
        return rc, rc2, data, dst, torch.equal(src, make(r, n))

    for rc, rc2, data, dst, src_intact in run_world(world, rank_fn):
        assert rc == 0 and rc2 == 0 and src_intact
        assert torch.allclose(data.double(), want, atol=2e-5)
        assert torch.equal(data, dst)


def test_single_rank_is_memcpy(env):
    def rank_fn(r, comm):
        a, b = torch.arange(10.0), torch.zeros(10)
        assert M.MPI_Allreduce_FT(a, b, 10, M.MPI_FLOAT, M.MPI_SUM, comm) == 0
        c = torch.arange(10.0)
        assert M.MPI_Allreduce_FT(M.IN_PLACE, c, 10, M.MPI_FLOAT, M.MPI_SUM, comm) == 0
        return b, c

    (b, c), = run_world(1, rank_fn)
    assert torch.equal(b, torch.arange(10.0)) and torch.equal(c, torch.arange(10.0))


def test_datatypes_and_band(env):
    env.pop("FT_TOPO", None); env.pop("FT_LONELY", None)
    cases = [(M.MPI_UINT8_T, torch.uint8), (M.MPI_INT8_T, torch.int8), (M.MPI_INT16_T, torch.int16), (M.MPI_INT32_T, torch.int32),
             (M.MPI_INT64_T, torch.int64), (M.MPI_LONG_LONG, torch.int64), (M.MPI_DOUBLE, torch.float64), (M.MPI_C_BOOL, torch.bool),
             (M.FT_BFLOAT16, torch.bfloat16), (M.FT_FLOAT16, torch.float16)]

    def rank_fn(r, comm):
        res = []
        for code, dt in cases:
            t = (torch.arange(50) % 3 == r % 3) if dt == torch.bool else torch.full((50,), r + 1).to(dt)
            rc = M.MPI_Allreduce_FT(M.IN_PLACE, t, 50, code, M.MPI_SUM, comm)
            res.append((rc, t))
        b = torch.full((9,), 0xFF ^ (1 << r), dtype=torch.int32)
        res.append((M.MPI_Allreduce_FT(M.IN_PLACE, b, 9, M.MPI_INT32_T, M.MPI_BAND, comm), b))
        return res

    out = run_world(4, rank_fn)
    for (code, dt), (rc, t) in zip(cases, out[0][:-1]):
        assert rc == 0
        if dt == torch.bool:
            assert bool(t.all())
        else:
            assert bool((t.double() == 10).all()), dt
    rc, b = out[2][-1]
    assert rc == 0 and bool((b == 0xF0).all())


def test_errors_are_returned_not_fatal(env, capfd):
    env["FT_TOPO"] = "2,3"
    env.pop("FT_LONELY", None)

    def bad_topo(r, comm):
        return M.MPI_Allreduce_FT(M.IN_PLACE, torch.zeros(4), 4, M.MPI_FLOAT, M.MPI_SUM, comm)

    assert run_world(4, bad_topo) == [4] * 4                      # 2*3 != 4 ranks
    assert "invalid FT_TOPO 2,3" in capfd.readouterr().err
    env.pop("FT_TOPO")

    def bad_type(r, comm):
        return (M.MPI_Allreduce_FT(M.IN_PLACE, torch.zeros(4), 4, M.MPI_FLOAT, M.MPI_BAND, comm),
                M.MPI_Allreduce_FT(M.IN_PLACE, torch.zeros(4), 4, M.MPI_FLOAT, M.MPI_MAX, comm),
                M.MPI_Allreduce_FT(M.IN_PLACE, torch.zeros(4), 4, 77, M.MPI_SUM, comm))

    assert run_world(2, bad_type) == [(2, 3, 2)] * 2
    err = capfd.readouterr().err
    assert "is not supported in MPI mode." in err and "Unsupported op 100" in err


def test_call_context_record_and_debug_print(env, capfd):
    """The per-call quantities the reference keeps in FlexTree_Context (mpi_mod.hpp:776-801): split size
    is ceil(count / N) whatever the tree, the aligned size is N splits; FT_DEBUG=1 prints them per call."""
    from allreduce_over_mpi_b200.parallel import planner as P
    c = P.context(7, 3, 27, torch.float32, lonely=1)
    assert c == {"num_nodes": 7, "node_label": 3, "num_lonely": 1, "data_size": 27, "num_split": 6, "split_size": 4,
                 "data_size_aligned": 28, "type_size": 4, "has_lonely": 1}
    assert P.context(10, 0, 1, torch.float64)["data_size_aligned"] == 10     # ten ranks, one element: nine empty blocks
    env["FT_TOPO"], env["FT_LONELY"], env["FT_DEBUG"] = "2,2", "1", "1"
    try:
        def rank_fn(r, comm):
            return M.MPI_Allreduce_FT(M.IN_PLACE, torch.ones(27), 27, M.MPI_FLOAT, M.MPI_SUM, comm)
        assert run_world(5, rank_fn) == [0] * 5
    finally:
        env.pop("FT_DEBUG", None)
    err = capfd.readouterr().err
    assert "num_nodes=5, node_label=4, num_lonely=1, data_size=27, num_split=4, split_size=6, data_size_aligned=30, type_size=4, has_lonely=1" in err


def test_debug_level_two_dumps_both_phases_in_rank_order(env, capfd):
    """FT_DEBUG=2: the call runs as reduce-scatter + all-gather and every rank prints the first values of its buffer
    after each half, rank after rank (the reference's "Med CHECK" / "Tail CHECK" dumps, mpi_mod.hpp:1601-1613,
    :1657-1670).  After the first half a rank's own block is complete; after the second everything is."""
    env["FT_TOPO"], env["FT_DEBUG"] = "2,2", "2"
    env.pop("FT_LONELY", None)
    try:
        bufs = {}

        def rank_fn(r, comm):
            bufs[r] = torch.full((8,), float(r + 1))
            return M.MPI_Allreduce_FT(M.IN_PLACE, bufs[r], 8, M.MPI_FLOAT, M.MPI_SUM, comm)
        assert run_world(4, rank_fn) == [0] * 4
    finally:
        env.pop("FT_DEBUG", None)
    assert all(bool((b == 10).all()) for b in bufs.values())
    lines = [l for l in capfd.readouterr().err.splitlines() if " CHECK node " in l]
    assert [l.split(":")[0] for l in lines] == [f"{tag} CHECK node {r}" for tag in ("Med", "Tail") for r in range(4)]
    for l in lines[:4]:      # blocks of two elements; rank r owns block r after the reduce-scatter
        r = int(l.split(":")[0].split()[-1])
        vals = [float(v) for v in l.split(":")[1].split()]
        assert vals[2 * r:2 * r + 2] == [10.0, 10.0]
    for l in lines[4:]:
        assert [float(v) for v in l.split(":")[1].split()] == [10.0] * 8
