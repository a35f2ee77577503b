"""Further multi-process, multi-GPU runs (one process per GPU under torch.distributed.run): the two halves of
the plan as collectives of their own, and data-parallel gradients against torch DDP over NCCL."""
import pytest

from test_comm_multigpu import ngpu, run_worker

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_reduce_scatter_and_all_gather_as_calls_of_their_own():
    n = min(ngpu(), 8)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    # with the two debugging aids on: guard blocks behind every heap tensor, collective symmetry check of alloc()
    res = run_worker(n, "phases", {"FT_CANARY": "1", "FT_CHECK_SYMMETRIC": "1"}, port=29581)
    assert res["ok"] and res["cases"] > 10 and res["guards_checked"] >= 1, res
    st = res["stats"]                     # every case is one reduce-scatter and one all-gather of the same bytes
    assert st["reduce_scatter"]["calls"] == st["all_gather"]["calls"] >= res["cases"]
    assert st["reduce_scatter"]["bytes"] == st["all_gather"]["bytes"] > 0


def test_ddp_gradients_equal_nccl_ddp():
    """One backward of a small GPT-2: FlexTreeDDP and the comm hook on torch DDP leave the same averaged
    gradients as torch DDP over NCCL."""
    n = min(ngpu(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    res = run_worker(n, "ddp", port=29591)
    assert res["ok"], res
    assert res["flextree_max_abs_err"] < 1e-4 and res["hook_max_abs_err"] < 1e-4


def test_split_optimizer_state_trains_like_nccl_ddp():
    """Three AdamW steps of a small GPT-2 with the optimizer's state split over the ranks (reduce-scatter of the
    gradients, all-gather of the parameters) end with the parameters torch DDP over NCCL gives with a whole AdamW per rank."""
    n = min(ngpu(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    res = run_worker(n, "zero", port=29595)
    assert res["ok"], res
    assert res["max_abs_err"] < 2e-5 and res["state_elements"] < res["params"] * 2


def test_a_rank_leaves_between_steps_and_the_survivors_carry_on():
    """Elastic recovery on GPUs without any GPU-side failure: a rank announces its departure on the host (a TCP store)
    before its last step, the others see it before their next launch, the old communicator is taken down by everyone
    together, and the survivors build a smaller communicator (new ranks, re-planned shape) and keep all-reducing.
    NVLS is off and no kernel ever waits for the rank that left."""
    n = min(ngpu(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    res = run_worker(n, "elastic", {"FT_NVLS": "0", "NCCL_NVLS_ENABLE": "0"}, port=29611)
    assert res["ok"], res
    assert res["new_world"] == n - 1 and res["lost"] == [res["leaver"]] and res["steps_before"] == 5 and res["steps_after"] == 5


def test_mpi_style_entry_on_gpu_communicators():
    """MPI_Allreduce_FT (the reference's entry point, mpi_mod.hpp:1723-1778) on GPU communicators: device buffers in and
    out of the heap, host buffers through the pipelined path, with the automatic choice and with FT_TOPO set; with
    FT_DEBUG=2 the call runs as its two halves and prints one value dump after each (mpi_mod.hpp:1601-1613, :1657-1670)."""
    n = min(ngpu(), 8)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    res = run_worker(n, "mpi", port=29601)
    assert res["ok"] and res["cases"] >= 40, res
    assert res["debug2"] == {"med": 1, "tail": 1}


def test_native_benchmark_checks_itself_on_gpus():
    """lib/ft_bench --comm-type flextree --check: ranks as threads of one process, heaps from the virtual-memory API,
    the algorithm chosen by the native policy."""
    import os
    import subprocess
    n = min(ngpu(), 8)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "allreduce_over_mpi_b200", "lib", "ft_bench")
    for size, extra in ((35, []), (1 << 22, []), (1 << 22, ["--dtype", "bf16"]), (1 << 20, ["--phases"])):
        r = subprocess.run([exe, "--gpus", str(n), "--size", str(size), "--repeat", "2", "--check", *extra], capture_output=True,
                           text=True, timeout=300)
        assert r.returncode == 0 and "CHECK (test passed)" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
