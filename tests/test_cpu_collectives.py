"""CPU correctness of every collective at world_size=2 (runs without a GPU): fp32 tensors of shape
[1024] and [3,1000] drawn from a seeded N(0,1), each result compared with plain torch math."""
import pytest
import torch
import torch.distributed as dist

from mp_util import run_ranks

SHAPES = [(1024,), (3, 1000)]


def _data(rank, shape, salt=0):
    g = torch.Generator().manual_seed(1234 + 17 * rank + salt)
    return torch.randn(*shape, generator=g)


def _all_reduce(rank, world):
    for shape in SHAPES:
        xs = [_data(r, shape) for r in range(world)]
        for op, ref in [(dist.ReduceOp.SUM, sum(xs)), (dist.ReduceOp.AVG, sum(xs) / world),
                        (dist.ReduceOp.MAX, torch.stack(xs).max(0).values),
                        (dist.ReduceOp.MIN, torch.stack(xs).min(0).values),
                        (dist.ReduceOp.PRODUCT, torch.stack(xs).prod(0))]:
            t = xs[rank].clone()
            dist.all_reduce(t, op=op)
            torch.testing.assert_close(t, ref, rtol=1e-6, atol=1e-6)


def _reduce_broadcast(rank, world):
    for shape in SHAPES:
        xs = [_data(r, shape) for r in range(world)]
        for root in range(world):
            t = xs[rank].clone()
            dist.reduce(t, dst=root, op=dist.ReduceOp.SUM)
            if rank == root:
                torch.testing.assert_close(t, sum(xs), rtol=1e-6, atol=1e-6)
            else:
                assert torch.equal(t, xs[rank])
        t = xs[rank].clone()
        dist.broadcast(t, src=0)
        assert torch.equal(t, xs[0])


def _gathers(rank, world):
    for shape in SHAPES:
        xs = [_data(r, shape) for r in range(world)]
        outs = [torch.empty(shape) for _ in range(world)]
        dist.all_gather(outs, xs[rank])
        for r in range(world):
            assert torch.equal(outs[r], xs[r])
        flat = torch.empty((world,) + shape)
        dist.all_gather_into_tensor(flat, xs[rank])
        assert torch.equal(flat, torch.stack(xs))
        g = [torch.empty(shape) for _ in range(world)] if rank == 0 else None
        dist.gather(xs[rank], g, dst=0)
        if rank == 0:
            for r in range(world):
                assert torch.equal(g[r], xs[r])
        out = torch.empty(shape)
        dist.scatter(out, xs if rank == 0 else None, src=0)
        ref0 = [_data(r, shape) for r in range(world)]
        assert torch.equal(out, ref0[rank])


def _reduce_scatter(rank, world):
    for shape in SHAPES:
        ins = [[_data(r, shape, salt=p) for p in range(world)] for r in range(world)]
        out = torch.empty(shape)
        dist.reduce_scatter(out, ins[rank])
        torch.testing.assert_close(out, sum(ins[r][rank] for r in range(world)), rtol=1e-6, atol=1e-6)
        flat_in = torch.cat([t.reshape(-1) for t in ins[rank]])
        out2 = torch.empty(flat_in.numel() // world)
        dist.reduce_scatter_tensor(out2, flat_in, op=dist.ReduceOp.AVG)
        ref = sum(torch.cat([t.reshape(-1) for t in ins[r]]) for r in range(world)) / world
        n = out2.numel()
        torch.testing.assert_close(out2, ref[rank * n:(rank + 1) * n], rtol=1e-6, atol=1e-6)


def _all_to_all(rank, world):
    # equal splits
    x = _data(rank, (world * 5, 7))
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x)
    ref = torch.cat([_data(r, (world * 5, 7))[rank * 5:(rank + 1) * 5] for r in range(world)])
    assert torch.equal(out, ref)
    # uneven splits: rank r sends r+1+p rows to rank p
    send = [[r + 1 + p for p in range(world)] for r in range(world)]
    xin = _data(rank, (sum(send[rank]), 3), salt=5)
    recv = [send[p][rank] for p in range(world)]
    out = torch.empty(sum(recv), 3)
    dist.all_to_all_single(out, xin, output_split_sizes=recv, input_split_sizes=send[rank])
    pieces = []
    for p in range(world):
        xp = _data(p, (sum(send[p]), 3), salt=5)
        off = sum(send[p][:rank])
        pieces.append(xp[off:off + send[p][rank]])
    assert torch.equal(out, torch.cat(pieces))
    # list version with uneven sizes
    ins = [_data(rank, (rank + p + 1,), salt=9) for p in range(world)]
    outs = [torch.empty(p + rank + 1) for p in range(world)]
    dist.all_to_all(outs, ins)
    for p in range(world):
        assert torch.equal(outs[p], _data(p, (p + rank + 1,), salt=9))


def _barrier_and_p2p(rank, world):
    dist.barrier()
    if rank == 0:
        dist.send(torch.arange(10.0), dst=1)
        t = torch.empty(300000)
        dist.recv(t, src=1)
        assert torch.equal(t, torch.arange(300000.0))
    else:
        t = torch.empty(10)
        dist.recv(t, src=0)
        assert torch.equal(t, torch.arange(10.0))
        dist.send(torch.arange(300000.0), dst=0)
    # both sides send first, then receive: must not deadlock
    peer = 1 - rank
    big = torch.full((1 << 20,), float(rank))
    got = torch.empty(1 << 20)
    ws = dist.isend(big, peer)
    wr = dist.irecv(got, peer)
    ws.wait()
    wr.wait()
    assert torch.all(got == float(peer))
    dist.barrier()


@pytest.mark.parametrize("fn", [_all_reduce, _reduce_broadcast, _gathers, _reduce_scatter, _all_to_all, _barrier_and_p2p],
                         ids=lambda f: f.__name__.strip("_"))
def test_cpu_world2(fn):
    run_ranks(fn, world=2)


def _dtype_matrix(rank, world):
    for dtype in [torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64, torch.float16, torch.bfloat16,
                  torch.float32, torch.float64]:
        x = (torch.arange(50) % 7 + rank + 1).to(dtype)
        ref = sum((torch.arange(50) % 7 + r + 1) for r in range(world)).to(dtype)
        t = x.clone()
        dist.all_reduce(t)
        assert torch.equal(t, ref), dtype
        if not dtype.is_floating_point:
            t = x.clone()
            dist.all_reduce(t, op=dist.ReduceOp.BXOR)
            r = torch.zeros(50, dtype=torch.int64)
            for k in range(world):
                r ^= (torch.arange(50) % 7 + k + 1)
            assert torch.equal(t, r.to(dtype)), dtype
    b = torch.tensor([rank == 0, True, False])
    dist.all_reduce(b, op=dist.ReduceOp.MAX)
    assert b.tolist() == [True, True, False]
    # large message: several shared-memory steps, two-shot schedule
    n = (9 << 20) // 4 + 3
    t = torch.full((n,), float(rank + 1))
    dist.all_reduce(t)
    assert torch.all(t == sum(range(1, world + 1)))


def test_cpu_dtypes_and_large_world3():
    run_ranks(_dtype_matrix, world=3)


def _edge_cases(rank, world):
    """Empty tensors, scalars, bool, non-contiguous input (refused like the reference:
    "input dense tensor has to be contiguous", src/utils.h check_tensor), object collectives."""
    t = torch.empty(0)
    dist.all_reduce(t)
    dist.all_gather([torch.empty(0) for _ in range(world)], t)
    dist.broadcast(t, 0)
    dist.all_to_all_single(torch.empty(0), t)
    dist.reduce_scatter_tensor(torch.empty(0), torch.empty(0))
    with pytest.raises(RuntimeError, match="contiguous"):
        dist.all_reduce(torch.ones(4, 4).t()[:, :2])
    s = torch.tensor(float(rank + 1))
    dist.all_reduce(s)
    assert s.item() == world * (world + 1) / 2
    b = torch.tensor([rank == 0, False])
    dist.all_reduce(b, op=dist.ReduceOp.MAX)
    assert b.tolist() == [True, False]
    objs = [None] * world
    dist.all_gather_object(objs, {"r": rank})
    assert [o["r"] for o in objs] == list(range(world))
    lst = [{"cfg": 7}] if rank == 0 else [None]
    dist.broadcast_object_list(lst, 0)
    assert lst == [{"cfg": 7}]


def test_edge_cases_world3():
    run_ranks(_edge_cases, world=3)


def _pending_works(rank, world):
    """waitForPendingWorks: after it returns, every Work issued before it is complete (collectives on the FIFO worker,
    sends and receives on their per-peer workers), without waiting on the Works one by one."""
    works, tensors = [], []
    for i in range(40):
        t = torch.full((4096,), float(rank + i))
        tensors.append(t)
        works.append(dist.all_reduce(t, async_op=True))
    peer = (rank + 1) % world
    if rank % 2 == 0:
        works.append(dist.isend(torch.arange(1000.0), peer))
    else:
        r = torch.empty(1000)
        tensors.append(r)
        works.append(dist.irecv(r, (rank - 1) % world))
    dist.group.WORLD._wait_for_pending_works()
    assert all(w.is_completed() for w in works)
    for i in range(40):
        assert torch.all(tensors[i] == float(sum(r + i for r in range(world))))
    if rank % 2 == 1:
        assert torch.equal(tensors[-1], torch.arange(1000.0))
    be = dist.group.WORLD._get_backend(torch.device("cpu"))
    be.wait_for_pending_works()  # nothing pending: returns at once
    dist.barrier()


def test_wait_for_pending_works_world2():
    run_ranks(_pending_works, world=2)
