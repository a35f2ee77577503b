"""Worker run under torch.distributed.run by test_comm_multigpu.py (one process per GPU)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from allreduce_over_mpi_b200.bench.allreduce import expected, fill, init_dist  # noqa: E402
from allreduce_over_mpi_b200.parallel import planner  # noqa: E402
from allreduce_over_mpi_b200.parallel.comm import FlexTreeComm  # noqa: E402


def elastic_main():
    """A rank leaves between steps; the survivors learn of it on the host before their next launch, take the old
    communicator down together with the leaver, form a smaller world and carry on.  Control traffic over gloo and a
    TCP store, NVLS off, no kernel ever waits for the rank that left."""
    import time
    from datetime import timedelta
    from allreduce_over_mpi_b200.parallel.elastic import Liveness, RankLost, replan_after_failure
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    port = int(os.environ["MASTER_PORT"])
    os.environ["FT_NVLS"] = "0"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo", rank=rank, world_size=world)       # rendezvous from the launcher's environment
    store = dist.TCPStore("127.0.0.1", port + 1, world, is_master=(rank == 0), timeout=timedelta(seconds=60))
    comm = FlexTreeComm(heap_bytes=32 << 20, staging_bytes=4 << 20, nvls=False, device=local)
    live = Liveness(store, rank, world, timeout_s=10.0)
    leaver, last_step = (world - 2 if world > 2 else 1), 4
    x = comm.alloc(1 << 16, torch.float32)
    report = {"world": world, "leaver": leaver, "steps_before": 0, "steps_after": 0}
    good = True
    plan = None
    try:
        for step in range(50):
            if rank == leaver and step == last_step:
                live.leave()                         # written before this rank's last launch
            live.guard()                             # between steps, before the next launch
            x.fill_(float(rank + 1))
            comm.all_reduce(x)
            torch.cuda.synchronize()
            comm.check()
            good = good and float(x[0]) == float(x[-1]) == world * (world + 1) / 2
            report["steps_before"] += 1
            if rank == leaver and step == last_step:
                break
    except RankLost as e:
        plan = replan_after_failure(world, e.lost, x.numel() * 4)
        report["lost"] = sorted(e.lost)
    # every rank of the old world, the leaver included, takes the old communicator down together: nobody maps the
    # leaver's heap any more when it exits
    comm.close()
    dist.destroy_process_group()
    if rank == leaver:
        good = good and report["steps_before"] == last_step + 1
        store.set(f"done/{rank}", json.dumps({"ok": bool(good), **report}))
        print(f"[rank {rank}] left after step {last_step}", flush=True)
        time.sleep(3.0)                              # the store's clients may still be reading
        return 0
    good = good and plan is not None and report.get("lost") == [leaver] and report["steps_before"] == last_step + 1
    new_rank, new_world = plan.rank_map[rank], plan.world
    # an explicit store: under torch.distributed.run a tcp:// or env:// rendezvous would look for the launcher's own store
    dist.init_process_group("gloo", store=dist.PrefixStore("survivors", store), rank=new_rank, world_size=new_world)
    comm = FlexTreeComm(heap_bytes=32 << 20, staging_bytes=4 << 20, nvls=False, device=local)
    y = comm.alloc(1 << 16, torch.float32)
    want = sum(r + 1 for r in range(world) if r != leaver)
    for _ in range(5):
        y.fill_(float(rank + 1))
        comm.all_reduce(y, shape=str(plan.shape))
        torch.cuda.synchronize()
        comm.check()
        good = good and float(y[0]) == float(y[-1]) == float(want)
        report["steps_after"] += 1
    report.update({"new_world": new_world, "new_rank": new_rank, "shape": str(plan.shape)})
    flags = [None] * new_world
    dist.all_gather_object(flags, bool(good))
    if new_rank == 0:
        print("RESULT " + json.dumps({"ok": all(flags), **report}), flush=True)
    comm.close()
    dist.destroy_process_group()
    if rank == 0:
        time.sleep(1.0)                              # rank 0 hosts the TCP store
    return 0 if all(flags) else 1


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "correctness"
    if mode == "elastic":
        return elastic_main()
    rank, world, local = init_dist()
    comm = FlexTreeComm(heap_bytes=96 << 20, staging_bytes=8 << 20, mem=os.environ.get("FT_MEM", "auto"))
    dev = comm.device
    report = {"world": world, "nvls": comm.has_nvls, "mem_kind": comm.mem_kind, "cases": 0}

    if mode == "timeout":
        # the last rank sits one call out; the others must come back with a timeout status, not hang
        comm.set_timeout_ms(300.0)
        x = torch.ones(4096, device=dev)
        comm.all_reduce(x, algo="oneshot")
        comm.check()
        if rank != world - 1:
            comm.all_reduce(x, shape=str(world), algo="staged")
            try:
                comm.check()
                report["timeout_seen"] = False
            except Exception as e:  # noqa: BLE001
                report["timeout_seen"] = "timeout" in str(e)
        else:
            report["timeout_seen"] = True
        torch.cuda.synchronize()
        flags = [None] * world
        dist.all_gather_object(flags, report["timeout_seen"])
        if rank == 0:
            print("RESULT " + json.dumps({"ok": all(flags), **report}), flush=True)
        comm.close()
        dist.destroy_process_group()
        return 0

    if mode == "ddp":
        # one backward of a small fp32 GPT-2 with rank-specific tokens: the gradients that FlexTreeDDP and the
        # FlexTree comm hook leave behind must equal those of torch DDP over NCCL (summation order aside)
        from torch.nn.parallel import DistributedDataParallel as DDP
        from allreduce_over_mpi_b200.models.gpt2 import GPT2, GPT2Config
        from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP, HookState, flextree_allreduce_hook
        cfg = GPT2Config.tiny()
        gen = torch.Generator().manual_seed(500 + rank)
        tok = torch.randint(0, cfg.vocab_size, (4, 33), generator=gen).to(dev)

        def grads(kind):
            torch.manual_seed(77)                      # same weights on every rank and in every arm
            model = GPT2(cfg).to(dev)
            comm.free_all()
            if kind == "flextree":
                wrap = FlexTreeDDP(model, comm, bucket_bytes=64 << 10)
            else:
                wrap = DDP(model, device_ids=[dev.index], bucket_cap_mb=1)
                if kind == "hook":
                    wrap.register_comm_hook(HookState(comm), flextree_allreduce_hook)
            loss = wrap(tok[:, :-1], tok[:, 1:])
            loss.backward()
            torch.cuda.synchronize()
            comm.check()
            flat = torch.cat([p.grad.detach().float().reshape(-1) for p in model.parameters()]).clone()
            return flat, float(loss.item())

        ref, loss_ref = grads("nccl")
        good = True
        for kind in ("flextree", "hook"):
            got, loss = grads(kind)
            err = (got - ref).abs().max().item()
            report[f"{kind}_max_abs_err"] = err
            if not err <= 1e-5 * max(1.0, ref.abs().max().item()) or abs(loss - loss_ref) > 1e-5:
                good = False
                print(f"[rank {rank}] {kind}: gradients differ from NCCL DDP by {err}, loss {loss} vs {loss_ref}", flush=True)
        report["cases"] = 2
        flags = [None] * world
        dist.all_gather_object(flags, good)
        if rank == 0:
            print("RESULT " + json.dumps({"ok": all(flags), **report}), flush=True)
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
        return 0 if all(flags) else 1

    if mode == "zero":
        # three AdamW steps of a small fp32 GPT-2 with rank-specific tokens: gradients reduce-scattered, optimizer state
        # split over the ranks, parameters all-gathered - against torch DDP over NCCL with a whole AdamW on every rank
        from torch.nn.parallel import DistributedDataParallel as DDP
        from allreduce_over_mpi_b200.models.gpt2 import GPT2, GPT2Config
        from allreduce_over_mpi_b200.parallel.ddp import FlexTreeDDP
        from allreduce_over_mpi_b200.parallel.zero import ShardedOptimizer
        cfg = GPT2Config.tiny()
        gen = torch.Generator().manual_seed(500 + rank)
        tok = torch.randint(0, cfg.vocab_size, (4, 33), generator=gen).to(dev)

        def make_opt(ps):
            return torch.optim.AdamW(ps, lr=1e-3, weight_decay=0.0)

        def train(kind):
            torch.manual_seed(77)
            model = GPT2(cfg).to(dev)
            comm.free_all()
            if kind == "sharded":
                wrap = FlexTreeDDP(model, comm, bucket_bytes=64 << 10, sharded=True)
                opt = ShardedOptimizer(wrap, make_opt)
            else:
                wrap = DDP(model, device_ids=[dev.index], bucket_cap_mb=1)
                opt = make_opt(model.parameters())
            losses = []
            for _ in range(3):
                opt.zero_grad()
                loss = wrap(tok[:, :-1], tok[:, 1:])
                loss.backward()
                opt.step()
                losses.append(float(loss.item()))
            torch.cuda.synchronize()
            comm.check()
            flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()]).clone()
            state = opt.state_elements() if kind == "sharded" else None
            return flat, losses, state

        ref, loss_ref, _ = train("nccl")
        got, loss_got, state = train("sharded")
        err = (got - ref).abs().max().item()
        nparam = ref.numel()
        report.update({"cases": 1, "max_abs_err": err, "loss_ref": loss_ref, "loss": loss_got, "state_elements": state, "params": nparam})
        good = err <= 2e-5 and all(abs(a - b) <= 1e-4 for a, b in zip(loss_got, loss_ref)) and state <= 2 * (nparam / world) * 1.5 + 4096
        # every rank must end with the same parameters, bit for bit
        mine = torch.tensor([float(got.double().sum().item())], device=dev, dtype=torch.float64)
        sums = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(sums, mine)
        good = good and all(bool((t == sums[0]).all()) for t in sums)
        flags = [None] * world
        dist.all_gather_object(flags, bool(good))
        if rank == 0:
            print("RESULT " + json.dumps({"ok": all(flags), **report}), flush=True)
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
        return 0 if all(flags) else 1

    if mode == "mpi":
        # the MPI-style C entry on a GPU communicator: device buffers (in and out of place, AUTO selection and an
        # explicit FT_TOPO), host buffers through the pipelined path, and the Python all_reduce_host
        import ctypes as C
        from allreduce_over_mpi_b200._lib import DTYPES, OPS, lib
        from allreduce_over_mpi_b200.parallel.mpi_compat import IN_PLACE
        L = lib()
        stream = torch.cuda.current_stream(dev).cuda_stream
        mc = L.ft_mpi_from_comm(comm._h, C.c_void_p(stream))
        good = True
        it = 0

        def close_enough(t, count, dtype, it_, what):
            nonlocal good
            want = expected(count, dtype, world, dev, it_)
            tol = 1e-4 if dtype == torch.float32 else 0.3
            err = (t.to(dev).double() - want).abs().max().item()
            if not err <= tol:
                good = False
                print(f"[rank {rank}] MPI_Allreduce_FT {what}: err {err}", flush=True)
            report["cases"] += 1

        explicit = {4: ("2,2", "0"), 5: ("2,2", "1"), 6: ("2,3", "0"), 7: ("2,3", "1"), 8: ("2,4", "0")}.get(world, (str(world), "0"))
        for topo in (None, explicit[0]):
            if topo is None:
                os.environ.pop("FT_TOPO", None)
                os.environ.pop("FT_LONELY", None)
            else:
                os.environ["FT_TOPO"], os.environ["FT_LONELY"] = explicit
            for dtype, name in ((torch.float32, "float32"), (torch.bfloat16, "bfloat16")):
                for count in (35, 70_001, (3 << 20) + 16):
                    it += 1
                    comm.free_all()
                    sym = comm.alloc(count, dtype)                 # device, heap resident, in place
                    fill(sym, rank, it)
                    rc = L.MPI_Allreduce_FT_c(IN_PLACE, sym.data_ptr(), count, DTYPES[name], OPS["sum"], mc)
                    torch.cuda.synchronize()
                    good = good and rc == 0
                    close_enough(sym, count, dtype, it, f"heap {topo} {name} {count}")
                    it += 1
                    src = torch.empty(count, dtype=dtype, device=dev)   # device, outside the heap, out of place
                    dst = torch.empty_like(src)
                    fill(src, rank, it)
                    rc = L.MPI_Allreduce_FT_c(src.data_ptr(), dst.data_ptr(), count, DTYPES[name], OPS["sum"], mc)
                    torch.cuda.synchronize()
                    good = good and rc == 0
                    close_enough(dst, count, dtype, it, f"device {topo} {name} {count}")
                    it += 1
                    fill(src, rank, it)
                    hsrc = src.cpu().pin_memory()                   # host buffers: pipelined through the GPU
                    hdst = torch.empty_like(hsrc).pin_memory()
                    rc = L.MPI_Allreduce_FT_c(hsrc.data_ptr(), hdst.data_ptr(), count, DTYPES[name], OPS["sum"], mc)
                    good = good and rc == 0
                    close_enough(hdst, count, dtype, it, f"host {topo} {name} {count}")
                    rc = L.MPI_Allreduce_FT_c(IN_PLACE, hsrc.data_ptr(), count, DTYPES[name], OPS["sum"], mc)
                    good = good and rc == 0
                    close_enough(hsrc, count, dtype, it, f"host in place {topo} {name} {count}")
        os.environ.pop("FT_TOPO", None)
        os.environ.pop("FT_LONELY", None)
        # a device tensor outside the heap that is larger than one staging slot is split natively
        it += 1
        big = torch.empty((comm.staging_bytes // 4) * 2 + 1000, dtype=torch.float32, device=dev)
        fill(big, rank, it)
        rc = L.MPI_Allreduce_FT_c(IN_PLACE, big.data_ptr(), big.numel(), DTYPES["float32"], OPS["sum"], mc)
        torch.cuda.synchronize()
        good = good and rc == 0
        close_enough(big, big.numel(), torch.float32, it, "larger than a slot")
        # Python front end of the pipelined host path, pageable memory too, averaged
        it += 1
        fill(big, rank, it)
        hp = big.cpu()
        out = comm.all_reduce_host(hp, out=torch.empty_like(hp), op="avg")
        torch.cuda.synchronize()
        close_enough(out * world, big.numel(), torch.float32, it, "all_reduce_host pageable avg")
        comm.check()
        # FT_DEBUG=2 on GPU ranks: the call runs as its two halves and prints the first 100 values after each
        # ("Med CHECK" after the reduce-scatter, "Tail CHECK" after the all-gather); the text goes to the C stderr,
        # which is pointed at a temporary file for the length of the call
        import tempfile
        it += 1
        comm.free_all()
        sym = comm.alloc(1000, torch.float32)
        fill(sym, rank, it)
        os.environ["FT_DEBUG"] = "2"
        with tempfile.TemporaryFile() as tf:
            sys.stderr.flush()
            saved = os.dup(2)
            os.dup2(tf.fileno(), 2)
            try:
                rc = L.MPI_Allreduce_FT_c(IN_PLACE, sym.data_ptr(), 1000, DTYPES["float32"], OPS["sum"], mc)
            finally:
                os.dup2(saved, 2)
                os.close(saved)
                os.environ.pop("FT_DEBUG", None)
            tf.seek(0)
            text = tf.read().decode(errors="replace")
        torch.cuda.synchronize()
        good = good and rc == 0
        close_enough(sym, 1000, torch.float32, it, "FT_DEBUG=2 halves")
        report["debug2"] = {"med": text.count("Med CHECK"), "tail": text.count("Tail CHECK")}
        if text.count("Med CHECK") != 1 or text.count("Tail CHECK") != 1:
            good = False
            print(f"[rank {rank}] FT_DEBUG=2 printed: {text[:300]!r}", flush=True)
        comm.check()
        L.ft_mpi_comm_free(mc)
        report["stats"] = comm.stats()
        flags = [None] * world
        dist.all_gather_object(flags, good)
        if rank == 0:
            print("RESULT " + json.dumps({"ok": all(flags), **report}), flush=True)
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
        return 0 if all(flags) else 1

    if mode == "phases":
        # reduce-scatter and all-gather as calls of their own: the owned block is complete after the
        # first, everything else is then overwritten with NaN, and the second alone rebuilds the result
        good = True
        it = 0
        for dtype in (torch.float32, torch.bfloat16):
            for count in (3, 4099, (3 << 20) + 5):
                for shape in [str(s) for s in planner.executable_shapes(world)]:
                    it += 1
                    comm.free_all()
                    sym = comm.alloc(count, dtype)
                    fill(sym, rank, it)
                    want = expected(count, dtype, world, dev, it)
                    tol = 1e-4 if dtype == torch.float32 else 0.3
                    owned = comm.reduce_scatter(sym, shape=shape)
                    torch.cuda.synchronize()
                    comm.check()
                    blocks = comm.owned_blocks(shape)
                    for b, view in zip(blocks, owned):
                        lo, hi = comm.block_range(sym, b)
                        if hi > lo and not (view.double() - want[lo:hi]).abs().max().item() <= tol:
                            good = False
                            print(f"[rank {rank}] reduce_scatter {shape} {dtype} {count}: block {b} is wrong", flush=True)
                    keep = [v.clone() for v in owned]
                    sym.fill_(float("nan"))
                    for v, k in zip(owned, keep):
                        v.copy_(k)
                    comm.all_gather(sym, shape=shape)
                    torch.cuda.synchronize()
                    comm.check()
                    if not (sym.double() - want).abs().max().item() <= tol:
                        good = False
                        print(f"[rank {rank}] all_gather {shape} {dtype} {count} is wrong", flush=True)
                    report["cases"] += 1
        # back to back without host synchronisation, the buffer rewritten between the calls
        comm.free_all()
        sym = comm.alloc(200_000, torch.float32)
        for i in range(8):
            sym.fill_(1.0)
            comm.reduce_scatter(sym, op="avg")
            comm.all_gather(sym)
        torch.cuda.synchronize()
        comm.check()
        good = good and bool(torch.allclose(sym, torch.ones_like(sym), atol=1e-5))
        sym.zero_()
        times = comm.profile_phases(sym, iters=3)
        comm.check()
        good = good and times["reduce_scatter_ms"] > 0 and times["all_gather_ms"] > 0
        report["phase_ms"] = times
        report["guards_checked"] = comm.check_canaries()     # > 0 when the test runs with FT_CANARY=1
        report["stats"] = comm.stats()
        flags = [None] * world
        dist.all_gather_object(flags, good)
        if rank == 0:
            print("RESULT " + json.dumps({"ok": all(flags), **report}), flush=True)
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
        return 0 if all(flags) else 1

    ok = True

    def verify(t, count, dtype, it, what):
        nonlocal ok
        torch.cuda.synchronize()
        comm.check()
        want = expected(count, dtype, world, dev, it)
        tol = 1e-4 if dtype == torch.float32 else 0.3
        err = (t.double() - want).abs().max().item()
        if not err <= tol:
            ok = False
            print(f"[rank {rank}] MISMATCH {what}: err {err}", flush=True)
        # every rank must hold the same bits
        h = t.view(torch.uint8).long().sum().reshape(1)
        lo, hi = h.clone(), h.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if lo.item() != hi.item():
            ok = False
            print(f"[rank {rank}] ranks disagree for {what}", flush=True)
        report["cases"] += 1

    shapes = [str(s) for s in planner.executable_shapes(world)]
    it = 0
    for dtype in (torch.float32, torch.bfloat16):
        for count in (1, 35, 4099, 1 << 20, (5 << 20) + 3):
            for shape in shapes:
                it += 1
                # tensor in the symmetric heap: in place, zero copy
                comm.free_all()
                sym = comm.alloc(count, dtype)
                fill(sym, rank, it)
                comm.all_reduce(sym, shape=shape, algo="staged")
                verify(sym, count, dtype, it, f"heap {shape} {dtype} {count}")
                # ordinary tensor: staged through the slots (split when larger than a slot)
                loc = torch.empty(count, dtype=dtype, device=dev)
                fill(loc, rank, it)
                comm.all_reduce(loc, shape=shape, algo="staged")
                verify(loc, count, dtype, it, f"slots {shape} {dtype} {count}")
            if count * 4 <= (64 << 10):
                for shape in shapes:     # the same plans on tagged words (no rendezvous), two calls each: both receive areas
                    for rep in range(2):
                        it += 1
                        loc = torch.empty(count, dtype=dtype, device=dev)
                        fill(loc, rank, it)
                        comm.all_reduce(loc, shape=shape, algo="ll")
                        verify(loc, count, dtype, it, f"tagged words {shape} {dtype} {count}")
            if count * 4 <= comm.staging_bytes:
                it += 1
                loc = torch.empty(count, dtype=dtype, device=dev)
                fill(loc, rank, it)
                comm.all_reduce(loc, algo="oneshot")
                verify(loc, count, dtype, it, f"oneshot {dtype} {count}")
            if count * loc.element_size() <= (256 << 10):
                for rep in range(3):   # consecutive calls alternate between the two receive areas
                    it += 1
                    loc = torch.empty(count, dtype=dtype, device=dev)
                    fill(loc, rank, it)
                    comm.all_reduce(loc, algo="ll")
                    verify(loc, count, dtype, it, f"ll {dtype} {count}")
            if comm.has_nvls and count * loc.element_size() <= comm.staging_bytes:
                for rep in range(2):   # one-shot through the switch: any tensor, odd lengths too; both staging slots
                    it += 1
                    loc = torch.empty(count, dtype=dtype, device=dev)
                    fill(loc, rank, it)
                    comm.all_reduce(loc, algo="nvls1")
                    verify(loc, count, dtype, it, f"nvls1 {dtype} {count}")
            if comm.has_nvls and (count * loc.element_size()) % 16 == 0:
                it += 1
                comm.free_all()
                sym = comm.alloc(count, dtype)
                fill(sym, rank, it)
                comm.all_reduce(sym, algo="nvls")
                verify(sym, count, dtype, it, f"nvls {dtype} {count}")
                for bf, lf in ((0.7, 0.5), (0.3, 0.25), (1.0, 0.9), (0.0, 0.1)):
                    it += 1
                    fill(sym, rank, it)
                    comm.set_hybrid(bf, lf)
                    comm.all_reduce(sym, algo="hybrid")
                    verify(sym, count, dtype, it, f"hybrid {bf}/{lf} {dtype} {count}")
            it += 1
            comm.free_all()
            sym = comm.alloc(count, dtype)
            fill(sym, rank, it)
            comm.all_reduce(sym, algo="push")
            verify(sym, count, dtype, it, f"push {dtype} {count}")
            it += 1
            comm.free_all()
            sym = comm.alloc(count, dtype)
            fill(sym, rank, it)
            comm.all_reduce(sym)      # cost model's pick
            verify(sym, count, dtype, it, f"auto {dtype} {count}")

    # back-to-back calls without host synchronisation: slots, call numbers and flags must keep up
    comm.free_all()
    count = 300_000
    sym = comm.alloc(count, torch.float32)
    loc = torch.empty(count, dtype=torch.float32, device=dev)
    small = torch.empty(1000, dtype=torch.float32, device=dev)
    sym.fill_(1.0); loc.fill_(1.0); small.fill_(1.0)
    rounds = 12
    for i in range(rounds):
        comm.all_reduce(sym, op="avg", shape=shapes[i % len(shapes)], algo="staged")
        comm.all_reduce(loc, op="avg", shape=shapes[(i + 1) % len(shapes)], algo="staged")
        comm.all_reduce(small, op="avg", algo="oneshot")
        comm.all_reduce(small, op="avg", algo="ll")
        comm.all_reduce(small, op="avg")
        comm.all_reduce(sym, op="avg", algo="push")
        if comm.has_nvls:
            comm.all_reduce(sym, op="avg", algo="nvls")
            comm.all_reduce(small, op="avg", algo="nvls1")
            comm.all_reduce(loc, op="avg", algo="nvls1")
    torch.cuda.synchronize()
    comm.check()
    for t, name in ((sym, "sym"), (loc, "loc"), (small, "small")):
        if not torch.allclose(t, torch.ones_like(t), atol=1e-5):
            ok = False
            print(f"[rank {rank}] back-to-back {name} drifted: {t[:4].tolist()}", flush=True)

    # CUDA graph: calls captured once and replayed (call numbers and slot parity live on the device)
    sym.fill_(1.0); small.fill_(1.0)
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        comm.all_reduce(sym, op="avg", shape=shapes[0], algo="staged")
        comm.all_reduce(small, op="avg", algo="ll")
        comm.all_reduce(small, op="avg", algo="oneshot")
        if comm.has_nvls:
            comm.all_reduce(sym, op="avg", algo="nvls")
            comm.all_reduce(small, op="avg", algo="nvls1")
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    comm.check()
    for t, name in ((sym, "sym"), (small, "small")):
        if not torch.allclose(t, torch.ones_like(t), atol=1e-5):
            ok = False
            print(f"[rank {rank}] graph replay {name} drifted: {t[:4].tolist()}", flush=True)
    report["graph_replays"] = 5

    # int32 sum and bitwise AND over the wire
    comm.free_all()
    xi = torch.full((10_001,), rank + 1, dtype=torch.int32, device=dev)
    comm.all_reduce(xi, shape=shapes[0], algo="staged")
    torch.cuda.synchronize()
    ok = ok and bool((xi == world * (world + 1) // 2).all())
    xb = torch.full((777,), 0x7fffffff ^ (1 << rank), dtype=torch.int32, device=dev)
    comm.all_reduce(xb, op="band", algo="oneshot")
    torch.cuda.synchronize()
    ok = ok and bool((xb == (0x7fffffff ^ ((1 << world) - 1))).all())

    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        print("RESULT " + json.dumps({"ok": all(flags), **report}), flush=True)
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0 if all(flags) else 1


if __name__ == "__main__":
    sys.exit(main())
