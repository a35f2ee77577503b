"""Calibration fit / choice table and re-planning after a lost rank (CPU)."""
import json

import torch

from allreduce_over_mpi_b200.parallel import planner, tune
from allreduce_over_mpi_b200.parallel.elastic import replan_after_failure
from allreduce_over_mpi_b200.parallel.planner import CostParams, Shape


def synth_rows(world=8, link=600.0, launch=20.0, sync=5.0):
    k = CostParams(launch_us=launch, sync_us=sync, link_gbs=link, stage_floor_us=0.0)
    rows = []
    for b in (1024, 1 << 20, 1 << 28):
        for shape in ("8", "2*4", "2*2*2"):
            us = planner.cost_v1(world, Shape.parse(shape), b, k)
            rows.append({"impl": f"flextree/staged/{shape}", "bytes": b, "world": world, "dtype": "float32", "ms": us / 1e3, "ok": True})
        rows.append({"impl": "flextree/nvls/auto", "bytes": b, "world": world, "dtype": "float32", "ms": (30 + b * 1.125 / 480e3) / 1e3})
        rows.append({"impl": "flextree/ll/auto", "bytes": b, "world": world, "dtype": "float32", "ms": (15 + b / 20e3) / 1e3})
        rows.append({"impl": "flextree/auto->nvls/8", "bytes": b, "world": world, "dtype": "float32", "ms": 1.0})
        rows.append({"impl": "nccl", "bytes": b, "world": world, "dtype": "float32", "ms": 1.0})
    return rows


def test_fit_recovers_the_generating_constants(tmp_path):
    rows = synth_rows()
    p, fit = tune.fit_params(rows)
    assert abs(p.link_gbs - 600) / 600 < 0.02
    assert abs(p.sync_us - 5.0) < 0.3 and abs(p.launch_us - 20.0) < 1.5
    assert 470 < p.nvls_gbs < 490
    assert max(abs(f["rel_err"]) for f in fit) < 0.05
    table = tune.best_table(rows)
    assert [r[1] for r in table["8"]] == ["ll", "nvls", "nvls"]
    # end to end through the command line, and the communicator-side loader
    src = tmp_path / "sweep.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in rows))
    out = tmp_path / "cal.json"
    assert tune.main([str(src), "--out", str(out)]) == 0
    assert planner.load_choice_table(out)["8"][0][1] == "ll"
    assert abs(CostParams.load(out).link_gbs - 600) < 15


def test_replan_after_failure_uses_lonely_layouts():
    r = replan_after_failure(8, {3}, 64 << 20, CostParams(link_gbs=600, sync_us=5, launch_us=20))
    assert r.world == 7 and r.rank_map == {0: 0, 1: 1, 2: 2, 4: 3, 5: 4, 6: 5, 7: 6}
    assert {"7", "2*3+1", "3*2+1", "ring7"} <= set(r.candidates)
    assert planner.validate_shape(7, r.shape) == "" and r.predicted_us > 0
    r = replan_after_failure(6, [0, 5], 1024)
    assert r.world == 4 and r.algo in ("oneshot", "staged", "ll")


def test_selection_from_the_committed_calibration():
    """What the communicator picks per message size on an 8-GPU box, from the committed table and model
    (pure host logic: no GPU is touched)."""
    from allreduce_over_mpi_b200.parallel.comm import _CommBase

    def comm(world, nvls):
        c = _CommBase()
        c.world, c.has_nvls, c.staging_bytes = world, nvls, 64 << 20
        return c

    c8 = comm(8, True)
    assert c8.choose(1024, True, torch.float32)[0] == "ll"
    assert c8.choose(1 << 30, True, torch.float32)[0] == "nvls"
    assert c8.choose(256 << 20, True, torch.bfloat16)[0] == "nvls"
    # integers, tensors outside the heap and boxes without multicast never get the switch reduction
    for args in ((1 << 30, True, torch.int32), (32 << 20, False, torch.float32)):
        assert c8.choose(*args)[0] not in ("nvls", "hybrid")
    name, shape = comm(8, False).choose(1 << 30, True, torch.float32)
    assert name in ("staged", "push") and planner.validate_shape(8, shape) == ""
    # outside the heap the in-place-only algorithms are out, and one-shot needs the message to fit a slot
    name, shape = c8.choose(32 << 20, False, torch.float32)
    assert name in ("staged", "oneshot") and planner.validate_shape(8, shape) == ""
    assert c8.choose(128 << 20, False, torch.float32)[0] == "staged"
    # without multicast nothing that needs the switch is ever picked, whatever the table says for the size
    for world in (4, 8):
        for nbytes in (1 << 20, 4 << 20, 256 << 20):
            assert comm(world, False).choose(nbytes, True, torch.float32)[0] not in ("nvls", "nvls1", "hybrid")
    # every world size from 2 to 8 gets a valid answer at every size, cached on the second ask
    for world in range(2, 9):
        c = comm(world, True)
        for nbytes in (16, 4096, 1 << 20, 48 << 20, 3 << 30):
            for in_heap in (True, False):
                name, shape = c.choose(nbytes, in_heap, torch.float32)
                assert name.split("-")[0] in ("ll", "oneshot", "staged", "push", "nvls", "nvls1", "hybrid")
                assert planner.validate_shape(world, shape) == ""
                assert c.choose(nbytes, in_heap, torch.float32) == (name, shape)


def test_heap_and_non_heap_tensors_of_one_size_do_not_share_a_cached_pick():
    """reduce+push works in place on heap tensors only: a pick cached for a heap tensor must never be handed to a
    tensor of the same size outside the heap (which would be refused at launch), nor the other way round."""
    from allreduce_over_mpi_b200.parallel.comm import _CommBase
    for world in (2, 3, 4):
        for first in (True, False):
            c = _CommBase()
            c.world, c.has_nvls, c.staging_bytes = world, False, 64 << 20
            for nbytes in (1 << 20, 16 << 20, 48 << 20):
                a = c.choose(nbytes, first, torch.float32)
                b = c.choose(nbytes, not first, torch.float32)
                fresh = _CommBase()
                fresh.world, fresh.has_nvls, fresh.staging_bytes = world, False, 64 << 20
                assert b == fresh.choose(nbytes, not first, torch.float32), (world, nbytes, first, a, b)
                outside = b if first else a
                assert outside[0] not in ("push", "nvls") and not outside[0].startswith("hybrid")


def test_native_policy_returns_every_row_of_the_committed_table(tmp_path):
    """The native policy (what ft_allreduce(FT_ALGO_AUTO), MPI_Allreduce_FT and ft_bench consult) answers each
    measured size of the committed calibration file with that row's winner; files that are not JSON are
    refused with a reason and leave the policy on the built-in model."""
    import ctypes as C
    import json
    from allreduce_over_mpi_b200._lib import Choice, lib
    L = lib()
    path = planner.calibration_path()
    table = json.load(open(path))["table"]
    assert table, "committed calibration has no table"
    for world_s, rows in table.items():
        world = int(world_s)
        h = L.ft_policy_create(world)
        err = C.create_string_buffer(256)
        assert L.ft_policy_load(h, path.encode(), err, 256) == 0 and err.value == b"", err.value
        assert L.ft_policy_num_rows(h) == len(rows)
        for r in rows:
            nbytes, algo, shape = r[0], r[1], r[2]
            out = Choice()
            assert L.ft_policy_choose(h, nbytes, 1, 1, 64 << 20, 8 << 10, 1, C.byref(out)) == 0
            assert out.from_table == 1
            assert out.algo_name.decode() == algo.split("-")[0], (world, r, out.algo_name)
            if algo == "staged":
                got = planner.Shape(tuple(out.widths[i] for i in range(out.nw)), out.lonely, bool(out.ring))
                assert str(got) == str(planner.Shape.parse(shape))
        L.ft_policy_destroy(h)
    bad = tmp_path / "broken.json"
    bad.write_text('{"params": {"launch_us": 3.0}, "table": {"8": [[1024, "ll", "8"],]}}')
    h = L.ft_policy_create(8)
    err = C.create_string_buffer(256)
    assert L.ft_policy_load(h, str(bad).encode(), err, 256) != 0 and b"offset" in err.value
    assert L.ft_policy_num_rows(h) == 0
    odd = tmp_path / "odd_rows.json"
    odd.write_text(json.dumps({"params": {"launch_us": 3.0, "peer_eff": {"2": 0.5}},
                               "table": {"8": [[1024, "ll", "8", 1.0], [4096, "warp-drive", "8"], [8192, "staged", "3*3"]]}}))
    assert L.ft_policy_load(h, str(odd).encode(), err, 256) == 0 and b"2 table rows skipped" in err.value
    assert L.ft_policy_num_rows(h) == 1
    # an "ll" row that names a tree keeps it: the plan then runs on tagged words
    L.ft_policy_clear_rows(h)
    assert L.ft_policy_add_row(h, 4096, b"ll", b"2*4") == 0 and L.ft_policy_add_row(h, 1 << 20, b"nvls", b"8") == 0
    assert L.ft_policy_add_row(h, 4096, b"ll", b"3*3") != 0          # not a shape of 8 ranks
    out = Choice()
    assert L.ft_policy_choose(h, 4096, 0, 0, 64 << 20, 8 << 10, 0, C.byref(out)) == 0
    assert out.algo_name == b"ll" and [out.widths[i] for i in range(out.nw)] == [2, 4] and out.from_table == 1
    from allreduce_over_mpi_b200._lib import V1Params
    k = V1Params()
    assert L.ft_policy_get_params(h, C.byref(k)) == 0 and k.launch_us == 3.0 and k.peer_eff[2] == 0.5
    L.ft_policy_destroy(h)


def _liveness_worker(rank, world, port, leave_after, q, session=None):
    import time
    import torch.distributed as dist
    from datetime import timedelta
    from allreduce_over_mpi_b200.parallel.elastic import Liveness, RankLost
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    live = Liveness(store, rank, world, timeout_s=1.5)   # generous: the ranks share a busy machine with other tests
    step = 0
    try:
        for step in range(500):
            if rank == leave_after[0] and step == leave_after[1]:
                q.put((rank, "left", step))
                time.sleep(6.0)      # stays quiet (keeps the process, and rank 0's store, alive) while the others notice
                return
            live.guard()              # between steps, before the next launch
            time.sleep(0.02)          # the step
        q.put((rank, "finished", step))
    except RankLost as e:
        plan = replan_after_failure(world, e.lost, 64 << 20, CostParams(link_gbs=600, sync_us=5, launch_us=20))
        q.put((rank, "lost", sorted(e.lost), plan.world, plan.rank_map[rank], str(plan.shape)))
        if session is not None:
            # the survivors form the smaller world under their new ranks and carry on with the re-planned shape
            from allreduce_over_mpi_b200.parallel.planner import ProcWorld
            w = ProcWorld(f"{session}-minus{len(e.lost)}", plan.rank_map[rank], plan.world, timeout_s=30)
            x = torch.full((1000,), float(rank + 1))          # 4 kB: travels through the control segment
            w.all_reduce(x, shape=plan.shape)
            q.put((rank, "recovered", float(x[0]), float(x[-1])))
            w.barrier()
            w.close()
        time.sleep(1.0)


def test_lost_rank_is_noticed_on_the_host_between_steps():
    """Three CPU processes around a TCP store; rank 2 stops stepping after step 10.  The other two learn
    of it from the store before a later step, agree on who is gone and on the plan for the smaller world."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    import socket
    with socket.socket() as sk:      # a port that is free right now
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    procs = [ctx.Process(target=_liveness_worker, args=(r, 3, port, (2, 10), q)) for r in range(3)]
    [p.start() for p in procs]
    got = [q.get(timeout=60) for _ in range(3)]
    [p.join(timeout=30) for p in procs]
    by_rank = {g[0]: g for g in got}
    assert by_rank[2][1] == "left"
    for r in (0, 1):
        assert by_rank[r][1] == "lost" and by_rank[r][2] == [2], by_rank
        assert by_rank[r][3] == 2 and by_rank[r][4] == r and by_rank[r][5] in ("2", "ring2")
    assert all(p.exitcode == 0 for p in procs)


def test_survivors_form_a_smaller_world_and_carry_on():
    """Four CPU processes; rank 1 goes quiet.  Ranks 0, 2 and 3 notice, re-plan for three ranks, join a new process world
    as ranks 0, 1, 2 and all-reduce there: the sum holds exactly the survivors' contributions."""
    import multiprocessing as mp
    import socket
    import uuid
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    session = "elastic-" + uuid.uuid4().hex[:10]
    procs = [ctx.Process(target=_liveness_worker, args=(r, 4, port, (1, 8), q, session)) for r in range(4)]
    [p.start() for p in procs]
    got = [q.get(timeout=90) for _ in range(7)]          # one "left", three "lost", three "recovered"
    [p.join(timeout=30) for p in procs]
    lost = {g[0]: g for g in got if g[1] == "lost"}
    rec = {g[0]: g for g in got if g[1] == "recovered"}
    assert sorted(lost) == sorted(rec) == [0, 2, 3], got
    assert [lost[r][4] for r in (0, 2, 3)] == [0, 1, 2] and all(lost[r][2] == [1] and lost[r][3] == 3 for r in lost)
    assert all(rec[r][2] == rec[r][3] == 1.0 + 3.0 + 4.0 for r in rec), rec
    assert all(p.exitcode == 0 for p in procs)


def test_liveness_in_one_process():
    import time
    import torch.distributed as dist
    from allreduce_over_mpi_b200.parallel.elastic import Liveness, RankLost
    store = dist.HashStore()
    a, b = Liveness(store, 0, 2, timeout_s=0.2), Liveness(store, 1, 2, timeout_s=0.2)
    for _ in range(5):
        a.guard(); b.guard()
        time.sleep(0.05)
    assert a.poll() == set()       # picks up b's last beat
    time.sleep(0.3)
    a.beat()                       # a keeps stepping, b has stopped
    assert a.poll() == {1}
    try:
        a.guard()
        raise AssertionError("expected RankLost")
    except RankLost as e:
        assert e.lost == {1}
    assert b.poll() == set()       # b still sees a's counter moving
    c, d = Liveness(dist.HashStore(), 0, 2, timeout_s=60.0), None
    d = Liveness(c.store, 1, 2, timeout_s=60.0)
    d.leave()                      # "my next step is my last": d's counter is 1, so that step is number 2
    d.guard()
    c.guard()                      # c's step 2: d still takes part in it
    try:
        c.guard()                  # c's step 3: d is gone, known at once, long before any silence would time out
        raise AssertionError("expected RankLost")
    except RankLost as e:
        assert e.lost == {1}


def test_fit_report_reads_the_committed_calibration():
    text = tune.report(planner.calibration_path())
    lines = text.splitlines()
    assert lines[0].startswith("cost model v1 fit:") and "| 8 |" in text and "fitted constants:" in text
    # every world size with several measured shapes reports how often the model's first choice was the fastest
    assert sum(" of " in l for l in lines if l.startswith("| ")) >= 5


def test_calibration_loader_survives_damaged_files(tmp_path):
    """Whatever is in the calibration file, loading returns a status: truncated, mutated and random files never crash the
    library, and a file that was refused leaves the policy answering from the built-in model."""
    import ctypes as C
    import random
    from allreduce_over_mpi_b200._lib import Choice, lib
    L = lib()
    good = open(planner.calibration_path(), "rb").read()
    rng = random.Random(12345)
    h = L.ft_policy_create(8)
    err = C.create_string_buffer(512)
    f = tmp_path / "cal.json"
    cases = [good[:n] for n in (0, 1, 17, len(good) // 3, len(good) - 1)]
    for _ in range(150):
        b = bytearray(good)
        for _ in range(rng.randint(1, 8)):
            i = rng.randrange(len(b))
            kind = rng.random()
            if kind < 0.4:
                b[i] = rng.randrange(256)
            elif kind < 0.7:
                del b[i:i + rng.randint(1, 40)]
            else:
                b[i:i] = bytes(rng.choice(b'{}[]",:0123456789eE+-.\\u') for _ in range(rng.randint(1, 12)))
        cases.append(bytes(b))
    cases += [bytes(rng.randrange(256) for _ in range(rng.randint(1, 300))) for _ in range(30)]
    cases += [b"[" * 5000, b'{"table": ' + b"[" * 3000, b'{"params": {"launch_us": 1e999}, "table": {"8": [[1e30, "ll", "8"]]}}']
    refused = 0
    for blob in cases:
        f.write_bytes(blob)
        rc = L.ft_policy_load(h, str(f).encode(), err, 512)
        refused += rc != 0
        out = Choice()
        assert L.ft_policy_choose(h, 1 << 20, 1, 0, 64 << 20, 8 << 10, 0, C.byref(out)) == 0
        assert out.algo_name.decode() in ("ll", "oneshot", "staged", "push", "nvls", "nvls1", "hybrid")
    assert refused > 10
    L.ft_policy_destroy(h)
