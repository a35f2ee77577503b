"""Planner + CPU executors.

Every executable shape for N <= 32 (flat, every ordered factorisation, ring, every valid
lonely layout) is run through the single-thread snapshot executor and checked against an
fp64 sum, for traffic optimality, fan-in bound and the static race check.  Invalid
layouts must be rejected with a message, never asserted or mis-scheduled.
"""

import pytest
import torch

from allreduce_over_mpi_b200.parallel import planner as P
from allreduce_over_mpi_b200.parallel.planner import Shape


def all_shapes(nmax):
    for n in range(1, nmax + 1):
        for s in P.executable_shapes(n):
            yield n, s


def make_bufs(world, count, dtype=torch.float32, seed=0):
    out = []
    for r in range(world):
        g = torch.Generator().manual_seed(seed * 1000 + r)
        x = torch.rand(count, generator=g, dtype=torch.float64) * 2 - 1
        out.append(x.to(dtype) if dtype.is_floating_point else (x * 100).to(dtype))
    return out


def test_shape_inventory():
    names = {n: [str(s) for s in P.executable_shapes(n)] for n in range(1, 11)}
    assert set(names[8]) >= {"8", "2*4", "4*2", "2*2*2", "ring8", "2*3+2", "3*2+2"}
    assert set(names[5]) >= {"5", "ring5", "2*2+1"}
    assert set(names[6]) >= {"6", "2*3", "3*2", "2*2+2"}
    assert set(names[7]) >= {"7", "2*3+1", "3*2+1"}
    # 3 ranks have no lonely form: a lonely layout needs at least two tree levels
    assert set(names[3]) == {"3", "ring3"}


@pytest.mark.parametrize("count", [1, 27, 1000])
def test_every_shape_up_to_32(count):
    checked = 0
    for n, s in all_shapes(32):
        assert P.validate_shape(n, s) == ""
        assert P.plan_check(n, s) == "", (n, str(s))
        bufs = make_bufs(n, count, torch.float64)
        want = torch.stack(bufs).sum(0)
        P.run_plan_snapshot(s, bufs)
        for r in range(n):
            assert torch.allclose(bufs[r], want, rtol=0, atol=1e-12), (n, str(s), r)
        assert P.plan_traffic(n, s, count) == 2 * (n - 1) * count, (n, str(s))
        assert P.plan_max_fanin(n, s) <= 32
        checked += 1
    assert checked > 300


def test_phases_alone_reduce_scatter_then_all_gather():
    """The two halves of every plan stand on their own: after the reduce-scatter half each block is
    complete on exactly the ranks rs_holders names (one per block), and the all-gather half reads
    nothing but those copies (every other block is poisoned before it runs)."""
    count = 53
    for n, s in all_shapes(16):
        holders = P.rs_holders(n, s)
        assert all(len(h) == 1 for h in holders), (n, str(s), holders)
        assert sorted(h[0] for h in holders) == list(range(n))       # every rank owns exactly one block
        bufs = make_bufs(n, count, torch.float64)
        want = torch.stack(bufs).sum(0)
        P.run_plan_snapshot(s, bufs, phase="reduce_scatter")
        B = -(-count // n)
        for b, (owner,) in enumerate(holders):
            lo, hi = min(count, b * B), min(count, (b + 1) * B)
            assert torch.allclose(bufs[owner][lo:hi], want[lo:hi], rtol=0, atol=1e-12), (n, str(s), b)
            assert P.owned_blocks(n, s, owner) == [b]
            for r in range(n):
                if r != owner:
                    bufs[r][lo:hi] = float("nan")
        P.run_plan_snapshot(s, bufs, phase="all_gather")
        for r in range(n):
            assert torch.allclose(bufs[r], want, rtol=0, atol=1e-12), (n, str(s), r)


def test_device_tables_pass_the_descriptor_check():
    """What the communicator verifies before it uploads a plan: every rank's table of every shape is
    in range (indices, block ids, fan-in, sources, and each stage reads only from ranks it has met)."""
    checked = 0
    for n, s in all_shapes(32):
        for r in range(n):
            assert P.dev_plan_check(n, s, r) == "", (n, str(s), r)
            checked += 1
    assert checked > 5000
    assert "rank" in P.dev_plan_check(4, Shape.flat(4), 9)
    assert P.dev_plan_check(7, Shape([2, 2], lonely=3), 0) != ""


def test_block_elems_matches_the_16_byte_rule():
    assert P.block_elems_for(1000, 8, 4) == 128          # ceil(1000/8) = 125 -> whole 16-byte vectors
    assert P.block_elems_for(1000, 8, 2) == 128
    assert P.block_elems_for(3, 8, 4) == 4
    assert P.block_elems_for(1 << 20, 7, 1) == 150016      # blocks of 64 KiB and more: whole multiples of 512 bytes
    assert P.block_elems_for(100_000, 7, 4) == 14288       # 57 KB blocks stay at 16-byte granularity


def test_lonely_validity_rule_is_exact():
    """L <= w0 and L*w0 <= M (with >= 2 levels) are accepted and correct; everything else is refused."""
    ok = bad = 0
    for n in range(3, 27):
        for l in range(1, 7):
            m = n - l
            if m < 2:
                continue
            for cand in P.candidate_shapes(m):
                w = tuple(int(x) for x in cand.split("*"))
                if 1 in w:
                    w = (m,)
                s = Shape(w, l)
                valid = len(w) >= 2 and l <= w[0] and l * w[0] <= m
                msg = P.validate_shape(n, s)
                assert (msg == "") == valid, (n, str(s), msg)
                if valid:
                    bufs = make_bufs(n, 101, torch.float64)
                    want = torch.stack(bufs).sum(0)
                    P.run_plan_snapshot(s, bufs)
                    assert all(torch.allclose(b, want, atol=1e-12) for b in bufs)
                    ok += 1
                else:
                    with pytest.raises(Exception):
                        P.run_plan_snapshot(s, make_bufs(n, 8, torch.float64))
                    bad += 1
    assert ok > 50 and bad > 50


def test_named_lonely_layouts():
    for text in ["2*2+1", "2*2+2", "2*3+1", "3*2+1", "2*2*2+1", "2*4+1", "4*2+1", "3*3+1", "2*2*2+2", "2*4+2",
                 "2*5+1", "3*3+2", "2*2*3+1", "3*2*2+1", "2*2*3+2", "2*2*2*2+1", "2*2*2*2+2"]:
        s = Shape.parse(text)
        for count in (3, 27, 101, 1000):
            bufs = make_bufs(s.world, count, torch.float64)
            want = torch.stack(bufs).sum(0)
            P.run_plan_snapshot(s, bufs)
            assert all(torch.allclose(b, want, atol=1e-12) for b in bufs), text


def test_golden_schedule_5_ranks():
    """5 = 2*2+1, 27 elements (blocks of 6, last block 24+3): who reads what from whom, per stage,
    must carry the same information as the reference planner's printed schedule."""
    s = Shape.parse("2*2+1")
    plan = P.plan_json(5, s)
    assert plan["stages"] == 4

    def pulls(rank, stage):
        return {(b, tuple(srcs)) for b, _red, srcs in plan["ranks"][rank][stage]["pulls"]}

    # RS stage 0: rank 0 (extended group with lonely rank 4) sums blocks 0,2 from ranks 1 and 4
    assert pulls(0, 0) == {(0, (1, 4)), (2, (1, 4))}
    assert pulls(1, 0) == {(1, (0, 4)), (3, (0, 4))}
    # rank 2 (non-extended, 2 % w0 == 0 < L) also collects the lonely block 4 from rank 3
    assert pulls(2, 0) == {(0, (3,)), (2, (3,)), (4, (3,))}
    assert pulls(3, 0) == {(1, (2,)), (3, (2,))}
    # the lonely rank gathers the lonely block from its adopted group {0,1}
    assert pulls(4, 0) == {(4, (0, 1))}
    # RS stage 1 (last): tree ranks finish their own block; rank 4 collects block 4 from holder 2
    assert pulls(0, 1) == {(0, (2,))} and pulls(2, 1) == {(2, (0,))}
    assert pulls(1, 1) == {(1, (3,))} and pulls(3, 1) == {(3, (1,))}
    assert pulls(4, 1) == {(4, (2,))}
    # AG stage 2 mirrors RS stage 1, AG stage 3 mirrors RS stage 0
    assert pulls(0, 2) == {(2, (2,))} and pulls(2, 2) == {(0, (0,)), (4, (4,))}
    assert pulls(4, 2) == set()
    assert pulls(0, 3) == {(1, (1,)), (3, (1,)), (4, (4,))}
    assert pulls(4, 3) == {(0, (0,)), (2, (0,)), (1, (1,)), (3, (1,))}
    assert pulls(3, 3) == {(0, (2,)), (2, (2,)), (4, (2,))}
    # element ranges in the text dump: block 4 is the short one
    text = P.describe(5, s, 4, count=27)
    assert "b4[24+3]" in text and "stage 0 RS" in text and "stage 3 AG" in text


def test_three_level_lonely_9():
    """9 = 2*2*2+1: block 8 follows star = 6; partials climb 5->4, 7->6, then 4->6, then 2,6 -> 8."""
    plan = P.plan_json(9, Shape.parse("2*2*2+1"))

    def lonely_pulls(rank, stage):
        return [tuple(srcs) for b, _r, srcs in plan["ranks"][rank][stage]["pulls"] if b == 8]

    assert lonely_pulls(8, 0) == [(0, 1)]
    assert lonely_pulls(2, 0) == [(3,)] and lonely_pulls(4, 0) == [(5,)] and lonely_pulls(6, 0) == [(7,)]
    assert lonely_pulls(6, 1) == [(4,)] and lonely_pulls(2, 1) == []
    assert lonely_pulls(8, 2) == [(6, 2)]


def test_ring_schedule():
    plan = P.plan_json(4, Shape.parse("ring4"))
    assert plan["stages"] == 6
    # rank 1 receives block 0 from its left neighbour first, then 3, then 2
    got = [plan["ranks"][1][s]["pulls"][0][0] for s in range(6)]
    assert got == [0, 3, 2, 1, 0, 3]
    assert all(plan["ranks"][1][s]["pulls"][0][2] == [0] for s in range(6))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64,
                                   torch.uint8, torch.int8, torch.int16, torch.float64])
def test_dtypes_sum(dtype):
    s = Shape.parse("2*3+1")
    bufs = make_bufs(7, 1234, dtype)
    want = torch.stack([b.double() for b in bufs]).sum(0)
    P.run_plan_snapshot(s, bufs)
    if dtype.is_floating_point:
        tol = {torch.float32: 1e-5, torch.float64: 1e-12, torch.bfloat16: 0.1, torch.float16: 0.02}[dtype]
        assert torch.allclose(bufs[0].double(), want, atol=tol)
    else:
        info = torch.iinfo(dtype)
        wrapped = want.long()
        if info.bits < 64:  # narrow integers wrap around like the native C++ addition
            span = info.max - info.min + 1
            wrapped = (wrapped - info.min) % span + info.min
        assert torch.equal(bufs[0].long(), wrapped)
    assert all(torch.equal(b, bufs[0]) for b in bufs)


def test_band_and_bool():
    s = Shape.parse("2*2")
    bufs = [torch.randint(0, 2 ** 31 - 1, (999,), dtype=torch.int32) for _ in range(4)]
    want = bufs[0] & bufs[1] & bufs[2] & bufs[3]
    P.run_plan_snapshot(s, bufs, op="band")
    assert all(torch.equal(b, want) for b in bufs)
    bb = [torch.rand(77) > 0.7 for _ in range(4)]
    want = bb[0] | bb[1] | bb[2] | bb[3]
    P.run_plan_snapshot(s, bb)
    assert all(torch.equal(b, want) for b in bb)
    with pytest.raises(Exception, match="unsupported type"):
        P.run_plan_snapshot(s, [torch.rand(8) for _ in range(4)], op="band")


def test_count_smaller_than_world():
    for text in ["8", "2*4", "2*2+1", "ring6"]:
        s = Shape.parse(text)
        for count in (1, 2, s.world - 1):
            bufs = make_bufs(s.world, count, torch.float64)
            want = torch.stack(bufs).sum(0)
            P.run_plan_snapshot(s, bufs)
            assert all(torch.allclose(b, want, atol=1e-12) for b in bufs)


def test_custom_block_size():
    s = Shape.parse("2*4")
    bufs = make_bufs(8, 1000, torch.float64)
    want = torch.stack(bufs).sum(0)
    P.run_plan_snapshot(s, bufs, block_elems=128)  # 8 * 128 >= 1000: last block short
    assert all(torch.allclose(b, want, atol=1e-12) for b in bufs)


def test_parse_topo_env_syntax():
    assert P.parse_topo(None, None, 8) == (Shape((8,)), False)
    assert P.parse_topo("", "", 6) == (Shape((6,)), False)
    assert P.parse_topo("2,3", None, 6) == (Shape((2, 3)), False)
    assert P.parse_topo("2,3", "1", 7) == (Shape((2, 3), 1), False)
    assert P.parse_topo("1", None, 5)[0].ring
    assert P.parse_topo("2,1,4", None, 5)[0].ring  # any width of 1 selects the ring
    assert P.parse_topo("auto", None, 8)[1] is True
    for topo, lonely, world in [("2,3", None, 7), ("2,2", "1", 6), ("6", "1", 7), ("2,2", "3", 7), ("3,2", "3", 9),
                                ("a,b", None, 4), ("2,4", "x", 10)]:
        with pytest.raises(Exception, match="invalid FT_"):
            P.parse_topo(topo, lonely, world)


def test_threaded_world_matches_oracle():
    for text in ["4", "2*2", "2*2+1", "ring5", "2*3+1", "2*2*2"]:
        s = Shape.parse(text)
        w = P.CpuWorld(s.world)
        for it in range(3):  # back-to-back calls reuse the flags with growing epochs
            bufs = make_bufs(s.world, 5000 + it, torch.float32, seed=it)
            want = torch.stack([b.double() for b in bufs]).sum(0)
            st = w.allreduce(s, bufs)
            assert all(x[0] == 0 for x in st), (text, st)
            assert all(torch.allclose(b.double(), want, atol=1e-5) for b in bufs)
        w.close()


def test_threaded_world_phases_as_calls_of_their_own():
    """Thread-per-rank world with the device protocol: reduce-scatter and all-gather as separate calls,
    each closed by an all-rank rendezvous, interleaved with whole all-reduces; the ranks poison what they
    do not own between the two halves, which is only safe because the closing rendezvous is global."""
    import threading
    for text in ["2", "ring3", "4", "2*2+1", "2*3+1", "2*2*2", "ring5", "2*4"]:
        s = Shape.parse(text)
        n, count = s.world, 4001
        w = P.CpuWorld(n, timeout_s=20)
        holders = P.rs_holders(n, s)
        B = -(-count // n)
        results, status = [None] * n, [[] for _ in range(n)]

        def rank_main(r):
            mine = [b for b, hs in enumerate(holders) if r in hs]
            for it in range(3):
                buf = make_bufs(n, count, torch.float64, seed=it)[r]
                status[r].append(w.phase_rank(r, s, buf, "reduce_scatter"))
                keep = {b: buf[min(count, b * B):min(count, (b + 1) * B)].clone() for b in mine}
                buf.fill_(float("nan"))
                for b, v in keep.items():
                    buf[min(count, b * B):min(count, (b + 1) * B)] = v
                status[r].append(w.phase_rank(r, s, buf, "all_gather"))
                status[r].append(w.allreduce_rank(r, s, buf))          # a whole call in between keeps the numbering honest
                results[r] = buf
        ts = [threading.Thread(target=rank_main, args=(r,)) for r in range(n)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        want = torch.stack(make_bufs(n, count, torch.float64, seed=2)).sum(0) * n
        for r in range(n):
            assert all(x[0] == 0 for x in status[r]), (text, r, status[r])
            assert torch.allclose(results[r], want, rtol=0, atol=1e-9), (text, r)
        w.close()


def test_fault_injection_on_host():
    """A rank that never signals / leaves early makes its peers time out; a wrong epoch is a protocol error."""
    s = Shape.parse("2*2")
    for kind, want_code in [(1, 5), (3, 5), (2, 8)]:
        w = P.CpuWorld(4, timeout_s=0.3)
        bufs = make_bufs(4, 64)
        st = w.allreduce(s, bufs, fault=(kind, 2, 1))  # rank 2 misbehaves at rendezvous 1
        codes = [x[0] for x in st]
        assert want_code in codes, (kind, st)
        bad = [x for x in st if x[0] == want_code]
        assert all(x[2] == 2 or x[0] == 5 for x in bad)  # the culprit is named (or a knock-on timeout)
        assert any(x[2] == 2 for x in bad)
        w.close()


def test_env_syntax_fuzz_never_yields_an_unusable_shape():
    """Whatever FT_TOPO / FT_LONELY hold, the parser either refuses with a message or returns a shape
    whose plan is race-free and sums correctly (the reference exits, asserts or mis-schedules on
    several of these, mpi_mod.hpp:1447-1475)."""
    from hypothesis import given, settings, strategies as st

    part = st.one_of(st.integers(-2, 12).map(str), st.sampled_from(["", " ", "a", "2x", "+1", "99999999999", "auto", "0"]))
    topo = st.lists(part, max_size=5).map(",".join)
    lonely = st.one_of(st.none(), st.integers(-3, 9).map(str), st.sampled_from(["", "x", "1.5", " 2"]))

    @settings(max_examples=400, deadline=None)
    @given(topo, lonely, st.integers(1, 24))
    def run(t, l, world):
        try:
            shape, is_auto = P.parse_topo(t, l, world)
        except Exception as e:  # noqa: BLE001
            assert "invalid FT_" in str(e), (t, l, world, str(e))
            return
        assert P.validate_shape(world, shape) == "", (t, l, world, str(shape))
        assert P.plan_check(world, shape) == ""
        bufs = make_bufs(world, 17, torch.float64)
        want = torch.stack(bufs).sum(0)
        P.run_plan_snapshot(shape, bufs)
        assert all(torch.allclose(b, want, rtol=0, atol=1e-12) for b in bufs), (t, l, world, str(shape))

    run()
