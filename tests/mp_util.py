"""Spawn helper for multi-process tests: runs `fn(rank, world, *args)` in `world` processes that
rendezvous through a FileStore (no network), and re-raises the first failure with its traceback.
Mirrors the reference's use of MultiProcessTestCase + FileStore (tests/test_c10d_ccl.py:95-103)."""
import os
import sys
import tempfile
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _entry(rank, world, fn, path, device, env, args, errq):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(env or {})
        os.environ.setdefault("OMP_NUM_THREADS", "1")
        torch.set_num_threads(1)
        import torch.distributed as dist

        import oneccl_bindings_for_pytorch  # noqa: F401

        if device == "cuda":
            torch.cuda.set_device(rank % torch.cuda.device_count())
        store = dist.FileStore(path, world)
        import datetime

        dist.init_process_group("ccl", store=store, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=float(os.environ.get("CCL_TEST_TIMEOUT_S", "60"))))
        try:
            fn(rank, world, *args)
        finally:
            if os.environ.get("CCL_TEST_NO_DESTROY") != "1":
                dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world=2, device="cpu", env=None, args=(), timeout=180):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_entry, args=(r, world, fn, path, device, env, args, errq)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        hung = [p for p in procs if p.is_alive()]
        for p in hung:
            p.kill()
        errs = []
        while not errq.empty():
            errs.append(errq.get())
        if errs:
            raise AssertionError("rank %d failed:\n%s" % errs[0])
        assert not hung, "ranks did not finish in time"
        bad = [p.exitcode for p in procs if p.exitcode != 0]
        assert not bad, f"ranks exited with {bad}"
