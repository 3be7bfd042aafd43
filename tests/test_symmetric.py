"""Symmetric tensors (memory of the communicator's heap that every rank maps) and the zero-copy collectives on them,
played on ONE GPU: one cooperative launch with gridDim.y == world runs every rank. Oracles: plain torch in fp64."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DT = [torch.bfloat16, torch.float16, torch.float32, torch.int32]


@pytest.fixture
def comm():
    import torch_ccl_b200._C as C

    made = []

    def make(world):
        c = C.CudaComm.emulated(world, 2 << 20, 2000, 8)
        c.set_symm_min_bytes(0)
        made.append(c)
        return c

    yield make
    torch.cuda.synchronize()
    made.clear()


def _symm(c, numel, dtype):
    """One symmetric tensor of `numel` elements per played rank."""
    return [t.view(dtype)[:numel] for t in c.symm_empty(numel * dtype.itemsize)]


def test_heap_allocator_is_deterministic_and_reuses_blocks(comm):
    c = comm(2)
    a = c.symm_empty(1000)
    b = c.symm_empty(5000)
    assert b[0].data_ptr() - a[0].data_ptr() == 1024  # rounded to 1 KB blocks, address order
    assert b[1].data_ptr() - a[1].data_ptr() == 1024  # same offsets in every rank's heap
    used = c.heap_in_use()
    pa = a[0].data_ptr()
    del a
    assert c.heap_in_use() == used - 1024
    d = c.symm_empty(512)
    assert d[0].data_ptr() == pa  # first fit: the hole is reused
    del b, d
    assert c.heap_in_use() == 0
    big = c.symm_empty(63 << 20)
    with pytest.raises(RuntimeError, match="exhausted"):
        c.symm_empty(2 << 20)
    del big


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("numel", [8, 4096, 100000 * 8])
def test_all_reduce_zero_copy(comm, world, dtype, numel):
    c = comm(world)
    torch.manual_seed(world + numel)
    xs = [(torch.randn(numel) * 3).to(dtype) for _ in range(world)]
    ins, outs = _symm(c, numel, dtype), _symm(c, numel, dtype)
    for it in range(2):  # out of place, then in place
        for r in range(world):
            ins[r].copy_(xs[r])
        dst = outs if it == 0 else ins
        tag = c.allreduce(ins, dst)
        torch.cuda.synchronize()
        assert c.status()[0] == 0, c.status()
        assert tag.split(":")[0] in ("nvls", "twoshot") and tag.endswith(":0"), tag  # took the symmetric kernels
        ref = torch.stack([x.double() for x in xs]).sum(0).to(dtype)
        tol = {torch.bfloat16: 2e-2, torch.float16: 4e-3, torch.float32: 1e-5, torch.int32: 0}[dtype]
        for r in range(world):
            torch.testing.assert_close(dst[r].cpu().double(), ref.double(), rtol=tol, atol=tol * world * 3)
            assert torch.equal(dst[r], dst[0])
    # MAX goes over the peer-load path (the switch only adds)
    for r in range(world):
        ins[r].copy_(xs[r])
    c.allreduce(ins, outs, op=3)
    torch.cuda.synchronize()
    assert torch.equal(outs[0].cpu(), torch.stack(xs).max(0).values)


def test_plain_tensors_still_take_the_staged_kernels(comm):
    c = comm(4)
    _ = c.symm_empty(1024)  # the heap exists, but these tensors are not in it
    xs = [torch.randn(4096, device="cuda") for _ in range(4)]
    outs = [torch.empty_like(x) for x in xs]
    tag = c.allreduce(xs, outs)
    torch.cuda.synchronize()
    assert not tag.endswith(":0")
    torch.testing.assert_close(outs[0], torch.stack(xs).sum(0), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
def test_reduce_scatter_zero_copy_with_cast_and_scale(comm, world, in_dtype, out_dtype):
    c = comm(world)
    n = 3000 * 8
    torch.manual_seed(9)
    full = [torch.randn(world * n).to(in_dtype) for _ in range(world)]
    ins = _symm(c, world * n, in_dtype)
    for r in range(world):
        ins[r].copy_(full[r])
    outs = [torch.empty(n, dtype=out_dtype, device="cuda") for _ in range(world)]
    before = c.launches
    c.reduce_scatter([list(t.chunk(world)) for t in ins], outs, 0, 1.0 / world, 1)
    torch.cuda.synchronize()
    assert c.status()[0] == 0 and c.launches == before + 1
    ref = torch.stack([f.double() for f in full]).sum(0) / world
    tol = 2e-2 if torch.bfloat16 in (in_dtype, out_dtype) else 1e-5
    for r in range(world):
        torch.testing.assert_close(outs[r].cpu().double(), ref[r * n:(r + 1) * n], rtol=tol, atol=tol * 4)


@pytest.mark.parametrize("world", [2, 8])
def test_all_gather_zero_copy(comm, world):
    c = comm(world)
    n = 5000 * 8
    pieces = [torch.randn(n).to(torch.bfloat16).cuda() for _ in range(world)]
    outs = _symm(c, world * n, torch.bfloat16)
    for _ in range(2):
        c.all_gather(pieces, [list(o.chunk(world)) for o in outs])
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    ref = torch.cat(pieces)
    for r in range(world):
        assert torch.equal(outs[r], ref)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.int32])
def test_batched_small_tensor_collectives(comm, world, dtype):
    """A list of tensors in ONE launch: all_reduce, reduce_scatter and all_gather over a pointer table."""
    c = comm(world)
    torch.manual_seed(world)
    sizes = [1, 7, 4096, 333, 8, 20003]
    data = [[(torch.randn(n) * 2).to(dtype) for n in sizes] for _ in range(world)]
    tol = {torch.bfloat16: 2e-2, torch.float32: 1e-5, torch.int32: 0}[dtype]
    before = c.launches
    # all_reduce (in place), averaged
    bufs = [[t.clone().cuda() for t in data[r]] for r in range(world)]
    scaled = dtype != torch.int32
    assert c.multi(0, bufs, bufs, 0, 1.0 / world if scaled else 1.0, 1 if scaled else 0)
    torch.cuda.synchronize()
    assert c.status()[0] == 0 and c.launches == before + 1
    for t, n in enumerate(sizes):
        ref = torch.stack([data[r][t].double() for r in range(world)]).sum(0) / (world if scaled else 1)
        for r in range(world):
            torch.testing.assert_close(bufs[r][t].cpu().double(), ref.to(dtype).double(), rtol=tol, atol=tol * world * 2)
    # reduce_scatter: every tensor holds `world` pieces
    full = [[(torch.randn(n * world) * 2).to(dtype) for n in sizes] for _ in range(world)]
    ins = [[t.cuda() for t in full[r]] for r in range(world)]
    outs = [[torch.empty(n, dtype=dtype, device="cuda") for n in sizes] for _ in range(world)]
    assert c.multi(1, ins, outs)
    torch.cuda.synchronize()
    for t, n in enumerate(sizes):
        ref = torch.stack([full[r][t].double() for r in range(world)]).sum(0).to(dtype)
        for r in range(world):
            torch.testing.assert_close(outs[r][t].cpu().double(), ref[r * n:(r + 1) * n].double(), rtol=tol, atol=tol * world * 2)
    # all_gather
    pieces = [[t.cuda() for t in data[r]] for r in range(world)]
    gathered = [[torch.empty(n * world, dtype=dtype, device="cuda") for n in sizes] for _ in range(world)]
    assert c.multi(2, pieces, gathered)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    for t, n in enumerate(sizes):
        ref = torch.cat([data[r][t] for r in range(world)])
        for r in range(world):
            assert torch.equal(gathered[r][t].cpu(), ref)
    # a list that is too large for the staging arena is refused, not truncated
    huge = [[torch.zeros(1 << 20, device="cuda")] * 4 for _ in range(world)]
    assert not c.multi(0, huge, huge)
