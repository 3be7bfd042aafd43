"""Bootstrap layer: descriptor exchange over UNIX sockets, symmetric memory through cudaIpc and
through driver virtual-memory objects, and the tuning file.

The reference's counterparts are hand-run native programs (src/test/segfault/simple_test.cpp,
src/test/writeremote/simple_test.cpp: map a peer's buffer through an IPC handle passed over a
UNIX socket, then read / write it) with print-and-eyeball checking; here the same steps are
asserted."""
import os

import pytest
import torch

from mp_util import run_ranks


def _fdx(rank, world):
    import torch.distributed as dist
    import torch_ccl_b200._C as C

    store = dist.distributed_c10d._get_default_store()
    for i in range(3):  # repeated exchanges use fresh socket names
        assert C.fd_exchange_probe(store, rank, world, "t/fdx/%d" % i)


def test_fd_exchange_world4():
    run_ranks(_fdx, world=4)


def test_fd_exchange_world1():
    run_ranks(_fdx, world=1)


def test_tune_text_parser():
    import torch_ccl_b200._C as C

    t = C.parse_tune_text("# measured on 8 GPUs\n8 oneshot_max_bytes=524288 max_blocks=128  # x\n\n2 threads=256 ag_push_max_bytes=0\n")
    assert t == {8: {"oneshot_max_bytes": 524288, "max_blocks": 128}, 2: {"threads": 256, "ag_push_max_bytes": 0}}
    t = C.parse_tune_text("4 nvls_min_bytes=8388608 symm_min_bytes=2097152 round_bytes=134217728 nvls_round_bytes=67108864 "
                          "ag_pull_round_bytes=33554432 ag_nvls_max_bytes=134217728\n")
    assert t[4]["nvls_round_bytes"] == 64 << 20 and t[4]["ag_pull_round_bytes"] == 32 << 20 and len(t[4]) == 6
    for bad, msg in [("8 foo=1", "unknown key"), ("9 threads=64", "world size"), ("8 threads=100", "out of range"),
                     ("8 threads", "key=value"), ("8", "no key=value"), ("8 threads=64\n8 threads=64", "twice"),
                     ("8 max_blocks=9999", "out of range"), ("x threads=64", "world size")]:
        with pytest.raises(RuntimeError, match=msg):
            C.parse_tune_text(bad)


def test_builtin_thresholds_follow_the_measured_tables():
    """The thresholds left to the library depend on the number of ranks: the values are the crossovers that the tuner
    and the sweep measured at 2, 4 and 8 GPUs. An explicit round size (CCL_ROUND_MB) also sets the two special cases."""
    import torch_ccl_b200._C as C

    t2, t4, t8 = (C.builtin_thresholds(w) for w in (2, 4, 8))
    assert t2["nvls_min_bytes"] > 1 << 50, "two ranks never pick the switch kernels by themselves"
    assert (t4["nvls_min_bytes"], t8["nvls_min_bytes"]) == (8 << 20, 2 << 20)
    assert (t2["symm_min_bytes"], t4["symm_min_bytes"], t8["symm_min_bytes"]) == (16 << 20, 2 << 20, 512 << 10)
    for t in (t2, t4, t8):
        assert (t["round_bytes"], t["nvls_round_bytes"], t["ag_pull_round_bytes"]) == (128 << 20, 64 << 20, 32 << 20)
        assert t["ag_nvls_max_bytes"] == 128 << 20
    e = C.builtin_thresholds(8, 16)
    assert (e["round_bytes"], e["nvls_round_bytes"], e["ag_pull_round_bytes"]) == (16 << 20, 16 << 20, 16 << 20)
    off = C.builtin_thresholds(4, 0)  # 0: rounds of the whole arena half
    assert (off["round_bytes"], off["nvls_round_bytes"], off["ag_pull_round_bytes"]) == (0, 0, 0)


def _symm(rank, world, kind):
    import torch.distributed as dist
    import torch_ccl_b200._C as C

    store = dist.distributed_c10d._get_default_store()
    assert C.symm_mem_probe(store, rank, world, kind, 3 << 20, "t/symm/" + kind)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["ipc", "vmm"])
def test_symm_mem_two_processes(kind):
    # both processes may share one GPU: the probe only copies, no kernel waits for another rank
    run_ranks(_symm, world=2, device="cuda", args=(kind,))


def _tuned(rank, world, path):
    import torch.distributed as dist

    x = torch.ones(1024, device="cuda")
    dist.all_reduce(x)
    assert torch.equal(x, torch.full_like(x, world))
    cfg = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cuda")).cuda_comm_config(x)
    assert cfg["oneshot_max_bytes"] == 12345 * 16 and cfg["threads"] == 256, cfg
    assert cfg["max_blocks"] == 64, cfg  # CCL_MAX_BLOCKS wins over the file's 32
    assert cfg["symm_mem"] == "vmm"
    be = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cuda"))
    be.set_cuda_tuning(x, {"oneshot_max_bytes": 1})  # same call on every rank: forces two-shot
    y = torch.full((1 << 16,), float(rank + 1), device="cuda")
    dist.all_reduce(y)
    assert torch.equal(y, torch.full_like(y, world * (world + 1) / 2))
    assert be.cuda_comm_config(x)["oneshot_max_bytes"] == 1


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_tune_file_and_vmm_arena_applied(tmp_path):
    world = 2
    p = tmp_path / "tune.txt"
    p.write_text("%d oneshot_max_bytes=%d threads=256 max_blocks=32\n" % (world, 12345 * 16))
    run_ranks(_tuned, world=world, device="cuda", args=(str(p),),
              env={"CCL_TUNE_FILE": str(p), "CCL_MAX_BLOCKS": "64", "CCL_SYMM_MEM": "vmm"})


def _nvls(rank, world):
    import torch.distributed as dist
    import torch_ccl_b200

    be = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cuda"))
    ok = True
    try:
        x = torch.ones(8, device="cuda")
        dist.all_reduce(x)  # creates the communicator (vmm arenas + multicast object)
        cfg = be.cuda_comm_config(x)
        assert cfg["symm_mem"] == "vmm" and cfg["nvls"]
        if not cfg["nvls_available"]:
            return  # no multicast support on this device: the plain kernels serve, nothing to check
        for dtype, n in [(torch.bfloat16, (4 << 20) + 24), (torch.float16, 3 << 20), (torch.float32, (2 << 20) + 1)]:
            t = ((torch.arange(n, device="cuda") % 13) + rank).to(dtype)
            dist.all_reduce(t)
            want = ((torch.arange(n, device="cuda") % 13) * world + world * (world - 1) // 2).to(dtype)
            assert torch.equal(t, want), (dtype, n, (t != want).sum().item())
        # reduce_scatter and all_gather through the same object (sizes above the 4 MB switch-over)
        n = 3 << 20
        full = ((torch.arange(n * world, device="cuda") % 11) + rank).to(torch.bfloat16)
        part = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(part, full)
        want = ((torch.arange(n * world, device="cuda") % 11) * world + world * (world - 1) // 2).to(torch.bfloat16)
        assert torch.equal(part, want[rank * n:(rank + 1) * n])
        gathered = torch.empty(n * world, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gathered, part)
        assert torch.equal(gathered, want)
        # broadcast above the switch-over: the root stores once into the multicast address (several rounds through
        # the 64 MB arena halves for the first tensor; an odd byte count for the second)
        root = world - 1
        big = torch.full((40 << 20,), rank + 1, device="cuda", dtype=torch.int32)
        dist.broadcast(big, src=root)
        assert int(big.min()) == root + 1 and int(big.max()) == root + 1
        odd = ((torch.arange((3 << 20) + 5, device="cuda") % 251) + (7 if rank == 0 else rank * 31)).to(torch.uint8)
        dist.broadcast(odd, src=0)
        assert torch.equal(odd, ((torch.arange((3 << 20) + 5, device="cuda") % 251) + 7).to(torch.uint8))
        t = torch.full((4 << 20,), float(rank + 1), device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
        assert torch.allclose(t, torch.full_like(t, (world + 1) / 2))
        torch.cuda.synchronize()
        assert "nvls" in torch_ccl_b200.flight_recorder()
    except BaseException:
        ok = False
        raise
    finally:
        # leave together and in order: nobody exits while a peer's memory is still bound
        torch.cuda.synchronize()
        store = dist.distributed_c10d._get_default_store()
        store.add("nvls_done", 1)
        import time

        t0 = time.time()
        while int(store.add("nvls_done", 0)) < world and time.time() - t0 < 20:
            time.sleep(0.01)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_switch_reduction_all_reduce():
    """CCL_NVLS=1: large SUM all_reduces go through the NVLink multicast object (multimem.ld_reduce
    + multimem.st); exact integer-valued inputs, so the result is compared bit for bit."""
    # two ranks never pick the switch kernels by themselves (they lose there): the threshold is given explicitly
    run_ranks(_nvls, world=min(torch.cuda.device_count(), 8), device="cuda",
              env={"CCL_NVLS": "1", "CCL_ARENA_MB": "64", "CCL_NVLS_MIN_BYTES": str(2 << 20)})


@pytest.mark.gpu
def test_single_rank_never_builds_a_multicast_object():
    import torch_ccl_b200._C as C

    torch.cuda.set_device(0)
    c = C.CudaComm.create(None, 0, 1, 8 << 20, 2000, "t/mc1", "vmm", True)
    assert not c.nvls_available
    x = torch.randn(1000, device="cuda")
    out = torch.zeros_like(x)
    assert not c.allreduce([x], [out], 0, 1.0, 0, 3).startswith("nvls")
    torch.cuda.synchronize()
    assert torch.equal(out, x)


def _symmetric_tensors(rank, world):
    """Tensors from the group's symmetric heap: collectives on them take the zero-copy kernels (through the
    switch when the heap is bound to a multicast object), plain tensors keep working next to them."""
    import time

    import torch.distributed as dist
    import torch_ccl_b200

    be = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cuda"))
    try:
        assert be.supports_tensor_alloc(torch.device("cuda", torch.cuda.current_device()))
        n = (1 << 20) + 8
        x = torch_ccl_b200.symm_empty(n, torch.bfloat16)
        y = torch_ccl_b200.symm_empty((2, n // 2), torch.float32)
        assert torch_ccl_b200.is_symmetric(x) and torch_ccl_b200.is_symmetric(y) and not torch_ccl_b200.is_symmetric(torch.ones(4, device="cuda"))
        info = be.symm_heap_info(x)
        assert info["in_use"] >= x.nbytes + y.nbytes
        for it in range(3):
            x.copy_(((torch.arange(n, device="cuda") % 13) + rank + it).to(torch.bfloat16))
            dist.all_reduce(x)
            want = ((torch.arange(n, device="cuda") % 13) * world + world * it + world * (world - 1) // 2).to(torch.bfloat16)
            assert torch.equal(x, want), (it, (x != want).sum().item())
        y.fill_(float(rank + 1))
        dist.all_reduce(y, op=dist.ReduceOp.AVG)
        assert torch.allclose(y, torch.full_like(y, (world + 1) / 2))
        z = torch.full((n,), float(rank), device="cuda")  # a plain tensor between symmetric ones
        dist.all_reduce(z)
        assert float(z[0]) == world * (world - 1) / 2
        # reduce_scatter from a symmetric input (bf16 -> bf16), all_gather into a symmetric output
        m = 1 << 18
        full = torch_ccl_b200.symm_empty(m * world, torch.bfloat16)
        full.copy_(((torch.arange(m * world, device="cuda") % 11) + rank).to(torch.bfloat16))
        part = torch.empty(m, device="cuda", dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(part, full)
        want = ((torch.arange(m * world, device="cuda") % 11) * world + world * (world - 1) // 2).to(torch.bfloat16)
        assert torch.equal(part, want[rank * m:(rank + 1) * m])
        gathered = torch_ccl_b200.symm_empty(m * world, torch.bfloat16)
        dist.all_gather_into_tensor(gathered, part)
        assert torch.equal(gathered, want)
        torch.cuda.synchronize()
        rec = torch_ccl_b200.flight_recorder()
        assert ("nvls" in rec) == bool(info["multicast"]), rec[-400:]
        # release in the same order on every rank; the blocks return to the heap
        del x, y, full, gathered
        torch_ccl_b200._C.drain()  # the watchdog keeps the tensors of in-flight work alive until it has retired them
        assert be.symm_heap_info(z)["in_use"] == 0
    finally:
        torch.cuda.synchronize()
        store = dist.distributed_c10d._get_default_store()
        store.add("symm_done", 1)
        t0 = time.time()
        while int(store.add("symm_done", 0)) < world and time.time() - t0 < 20:
            time.sleep(0.01)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("nvls", ["0", "1"])
def test_symmetric_tensors_zero_copy(nvls):
    run_ranks(_symmetric_tensors, world=min(torch.cuda.device_count(), 8), device="cuda",
              env={"CCL_NVLS": nvls, "CCL_ARENA_MB": "64", "CCL_SYMM_HEAP_MB": "64", "CCL_SYMM_MIN_BYTES": "0", "NCCL_NVLS_ENABLE": "0"})
