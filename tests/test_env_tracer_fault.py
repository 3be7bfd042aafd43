"""Environment knobs, the verbose tracer's line format, statistics / flight recorder, and
host-side failure detection (a rank that never joins a collective; a rank that leaves between
steps). No GPU is faulted or hung anywhere: failures are made on the host (CPU ranks; on GPUs a rank that
does not join one collective, which its peer's kernel answers with a bounded wait and a status word)."""
import os
import re
import subprocess
import sys
import time

import pytest
import torch
import torch.distributed as dist

from mp_util import ROOT, run_ranks


def _run_py(code, env=None):
    e = dict(os.environ)
    e.update(env or {})
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    return subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=120)


def test_env_flag_parsing_rules():
    code = "import oneccl_bindings_for_pytorch as c, torch_ccl_b200._C as C; print(C.env())"
    r = _run_py(code, {"CCL_BLOCKING_WAIT": "1", "CCL_SAME_STREAM": "0", "TORCH_LLM_ALLREDUCE": "1", "CCL_ARENA_MB": "32",
                       "LOCAL_RANK": "3", "LOCAL_WORLD_SIZE": "8"})
    assert r.returncode == 0, r.stderr
    env = eval(r.stdout.strip().splitlines()[-1])
    assert env["blocking_wait"] is True
    assert env["same_stream"] is True  # implied by TORCH_LLM_ALLREDUCE
    assert env["arena_mb"] == 32 and env["local_rank"] == 3 and env["local_world_size"] == 8
    # "2" is an integer but not 1 -> false; a non-integer is an error naming the variable
    r = _run_py(code, {"CCL_BLOCKING_WAIT": "2"})
    assert eval(r.stdout.strip().splitlines()[-1])["blocking_wait"] is False
    r = _run_py(code, {"CCL_BLOCKING_WAIT": "yes"})
    assert r.returncode != 0 and "Invalid value for environment variable: CCL_BLOCKING_WAIT" in r.stderr
    r = _run_py(code, {"PMI_RANK": "0", "MPI_LOCALRANKID": "1", "MPI_LOCALNRANKS": "2"})
    env = eval(r.stdout.strip().splitlines()[-1])
    assert env["with_mpirun"] is True and env["local_rank"] == 1 and env["local_world_size"] == 2


def _traced(rank, world):
    t = torch.zeros(3, 1000)
    dist.all_reduce(t)
    dist.broadcast(t, src=1)
    dist.reduce(t, dst=0)
    dist.barrier()


def test_verbose_tracer_line_format(capfd):
    run_ranks(_traced, world=2, env={"ONECCL_BINDINGS_FOR_PYTORCH_ENV_VERBOSE": "1"})
    out = capfd.readouterr().out
    # header line, then the same line with the elapsed time appended (reference: dispatch_stub.cpp:61-119)
    assert re.search(r"oneccl_bindings_for_pytorch::cpu::allreduce: \[0/2#\d+\] \[\(cpu, \[3, 1000\]\)\]\n", out)
    assert re.search(r"oneccl_bindings_for_pytorch::cpu::allreduce: \[1/2#\d+\] \[\(cpu, \[3, 1000\]\)\] Time elapsed \(ms\): [\d.e+-]+", out)
    assert re.search(r"oneccl_bindings_for_pytorch::cpu::broadcast: \[0/2#\d+\] \[1->0\] ", out)
    assert re.search(r"oneccl_bindings_for_pytorch::cpu::reduce: \[1/2#\d+\] \[1->0\] ", out)


def _stats(rank, world):
    import torch_ccl_b200 as ccl

    ccl._C.reset_stats()
    for _ in range(5):
        dist.all_reduce(torch.ones(256))
    dist.barrier()
    st = ccl.stats()
    assert st["cpu::allreduce"]["count"] == 5 and st["cpu::allreduce"]["bytes"] == 5 * 1024
    assert sum(st["cpu::allreduce"]["host_us_hist"]) == 5
    fr = ccl.flight_recorder()
    assert "cpu::allreduce bytes=1024" in fr and "NOT COMPLETED" not in fr.split("barrier")[0]


def test_stats_and_flight_recorder():
    run_ranks(_stats, world=2)


def _missing_rank(rank, world):
    dist.barrier()
    t = torch.ones(4)
    if rank == 1:
        time.sleep(4.0)  # never joins the collective in time
        return
    t0 = time.time()
    with pytest.raises(dist.DistBackendError, match="Caught collective operation timeout"):
        dist.all_reduce(t)
    assert time.time() - t0 < 3.5, "the wait must be bounded by the group timeout"
    pg = dist.group.WORLD._get_backend(torch.device("cpu"))
    assert pg.error_state() != 0
    assert "allreduce" in __import__("torch_ccl_b200").flight_recorder()


def test_rank_that_never_joins_times_out_on_peers():
    run_ranks(_missing_rank, world=2, env={"CCL_TEST_TIMEOUT_S": "1.5", "CCL_TEST_NO_DESTROY": "1"})


def test_bring_up_without_the_peer_fails_with_a_named_count():
    """Bootstrap failure made on the host: rank 0 of a two-rank group runs alone (its peer never starts). The first CPU
    collective builds the communicator, waits CCL_INIT_TIMEOUT_MS for the other rank and fails with a DistBackendError that
    says how many ranks showed up; nothing hangs."""
    code = (
        "import datetime, os, sys, tempfile, time\n"
        "import torch, torch.distributed as dist\n"
        "import oneccl_bindings_for_pytorch\n"
        "store = dist.FileStore(os.path.join(tempfile.mkdtemp(), 's'), 2)\n"
        "dist.init_process_group('ccl', store=store, rank=0, world_size=2, timeout=datetime.timedelta(seconds=2))\n"
        "t0 = time.time()\n"
        "try:\n"
        "    dist.all_reduce(torch.ones(4))\n"
        "    print('NO ERROR')\n"
        "except dist.DistBackendError as e:\n"
        "    print('RAISED %.1f %s' % (time.time() - t0, e))\n"
        "os._exit(0)\n"
    )
    r = _run_py(code, env={"CCL_INIT_TIMEOUT_MS": "1500"})
    assert r.returncode == 0, r.stderr[-2000:]
    assert "RAISED" in r.stdout and "1 of 2 ranks" in r.stdout, r.stdout + r.stderr[-2000:]
    assert float(r.stdout.split("RAISED ")[1].split()[0]) < 10


def _watchdog_deadline_cuda(rank, world):
    """Rank 1 does not join one all_reduce. Rank 0's kernel waits for it with a budget of 12 s (set far above the
    group's timeout of 3 s on purpose), so only the watchdog's own deadline can end the work early: it raises the
    communicator's abort word, the kernel's wait samples it and returns with status 'aborted', the context stays
    usable. Rank 1 leaves after rank 0 has seen the failure, with no kernel of its own in flight."""
    import datetime

    t = torch.ones(1 << 16, device="cuda")
    dist.all_reduce(t)
    torch.cuda.synchronize()
    store = dist.distributed_c10d._get_default_store()
    if rank != 0:
        store.wait(["watchdog_seen"], datetime.timedelta(seconds=60))
        return
    t0 = time.time()
    try:
        w = dist.all_reduce(t, async_op=True)
        while not w.is_completed() and time.time() - t0 < 40:
            time.sleep(0.05)
        dt = time.time() - t0
        time.sleep(0.5)  # the watchdog retires the work right after the event fires
        with pytest.raises(dist.DistBackendError, match="abort"):
            w.wait()
        assert 3.0 < dt < 10.5, dt
        torch.cuda.synchronize()  # the context survived
        assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
        with pytest.raises(dist.DistBackendError):
            dist.all_reduce(t)  # the communicator stays failed
    finally:
        store.set("watchdog_seen", "1")


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_watchdog_deadline_aborts_a_work_past_its_timeout():
    run_ranks(_watchdog_deadline_cuda, world=2, device="cuda",
              env={"CCL_TEST_TIMEOUT_S": "3", "CCL_SPIN_TIMEOUT_MS": "12000", "CCL_TEST_NO_DESTROY": "1",
                   "NCCL_NVLS_ENABLE": "0", "CCL_NVLS": "0"})


def _leaves_between_steps(rank, world):
    """Elastic pattern: a rank leaves between steps; the survivors learn of it on the host (store
    heartbeat) before their next collective, drop the group and build a smaller one."""
    store = dist.distributed_c10d._get_default_store()
    for step in range(3):
        t = torch.ones(8)
        dist.all_reduce(t)
        assert torch.all(t == world)
    if rank == world - 1:
        store.set("left", str(rank))
        return
    store.wait(["left"])
    gone = int(store.get("left"))
    survivors = [r for r in range(world) if r != gone]
    import oneccl_bindings_for_pytorch  # noqa: F401

    sub = dist.ProcessGroupCCL(dist.PrefixStore("regroup", store), survivors.index(rank), len(survivors))
    t = torch.ones(8)
    sub.allreduce([t]).wait()
    assert torch.all(t == len(survivors))
    sub.shutdown()


def test_regroup_after_a_rank_leaves():
    run_ranks(_leaves_between_steps, world=3, env={"CCL_TEST_NO_DESTROY": "1"})


def _mismatched(rank, world):
    """CCL_DEBUG_CHECKS=1: ranks that call different collectives get an error naming both sides."""
    t = torch.ones(8)
    dist.all_reduce(t)  # matching call passes
    assert torch.all(t == world)
    with pytest.raises(dist.DistBackendError, match="collective mismatch at collective #1.*8 bytes.*64 bytes|collective mismatch at collective #1.*64 bytes.*8 bytes"):
        dist.all_reduce(torch.ones(2 if rank == 0 else 16))
    with pytest.raises(dist.DistBackendError, match="collective mismatch"):
        if rank == 0:
            dist.broadcast(torch.ones(4), 0)
        else:
            dist.all_reduce(torch.ones(4))
    with pytest.raises(dist.DistBackendError, match="collective mismatch.*Float.*Double|collective mismatch.*Double.*Float"):
        dist.all_reduce(torch.ones(4, dtype=torch.float32 if rank == 0 else torch.float64))
    # uneven all_to_all legitimately differs in size per rank: only the op and dtype are compared
    ins = torch.arange(rank + 1 + world - 1, dtype=torch.float32)
    in_split = [rank + 1] + [1] * (world - 1)
    out_split = [p + 1 for p in range(world)] if rank == 0 else [1] * world
    out = torch.empty(sum(out_split))
    dist.all_to_all_single(out, ins, out_split, in_split)
    assert out.numel() == (world * (world + 1) // 2 if rank == 0 else world)
    # point-to-point traffic between two collectives does not disturb the counter
    if rank == 0:
        dist.send(torch.ones(3), 1)
    elif rank == 1:
        dist.recv(torch.empty(3), 0)
    dist.all_reduce(t)


def test_debug_checks_name_mismatched_collectives():
    run_ranks(_mismatched, world=2, env={"CCL_DEBUG_CHECKS": "1", "CCL_TEST_TIMEOUT_S": "20"})
