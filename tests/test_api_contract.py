"""API-level contract of the backend on CPU ranks: direct ProcessGroupCCL construction, error
strings, root validation, async stress, coalescing manager, _broadcast_coalesced, DDP, sub-groups,
object collectives. Mirrors the cases of the reference's tests/test_c10d_ccl.py (broadcast root
checks :109-113, 1000-op stress :152-171, allgather_base errors :377-440, coalescing :666-733,
_broadcast_coalesced :735-763) with the missing waits and assertions added."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist

from mp_util import run_ranks


def test_import_registers_backend_and_attributes():
    import oneccl_bindings_for_pytorch as ccl
    import torch_ccl

    assert dist.is_backend_available("ccl")
    assert hasattr(dist, "ProcessGroupCCL")
    assert ccl.__version__.startswith("2.8.0") and isinstance(ccl.git_version, str) and os.path.isdir(ccl.cwd)
    a, b = torch.zeros(4), torch.zeros(4, 4).t()
    assert ccl.is_available([a]) and not ccl.is_available([b])
    assert not ccl.is_available([a, a.clone()])  # same device twice
    assert torch_ccl.is_available([a])


def test_world1_direct_construction_and_noop_collectives():
    import oneccl_bindings_for_pytorch  # noqa: F401

    with tempfile.TemporaryDirectory() as d:
        store = dist.FileStore(os.path.join(d, "s"), 1)
        pg = dist.ProcessGroupCCL(store, 0, 1)
        assert pg.name() == "ccl" if hasattr(pg, "name") else True
        t = torch.arange(6.0)
        w = pg.allreduce([t])
        w.wait()
        assert torch.equal(t, torch.arange(6.0))
        assert w.is_completed() and w.is_success()
        assert torch.equal(w.result()[0], t)
        out = torch.empty(6)
        pg._allgather_base(out, t).wait()
        assert torch.equal(out, t)
        pg.barrier().wait()
        pg.shutdown()


def _errors(rank, world):
    pg = dist.group.WORLD._get_backend(torch.device("cpu"))
    t = torch.zeros(8)
    for bad in (-1, world):
        o = dist.BroadcastOptions()
        o.rootRank = bad
        with pytest.raises(ValueError, match="unexpected rank"):
            pg.broadcast([t], o)
        r = dist.ReduceOptions()
        r.rootRank = bad
        with pytest.raises(ValueError, match="unexpected rank"):
            pg.reduce([t], r)
    with pytest.raises(RuntimeError, match="does not support tensors count 2"):
        pg.allreduce([t, t.clone()])
    with pytest.raises(RuntimeError, match="input dense tensor has to be contiguous"):
        pg.allreduce([torch.zeros(4, 4).t()])
    with pytest.raises(RuntimeError, match="output tensor size must be equal to world_size times input tensor size"):
        pg._allgather_base(torch.empty(8 * world + 1), t)
    with pytest.raises(RuntimeError, match="output tensor must have the same type as input tensor"):
        pg._allgather_base(torch.empty(8 * world, dtype=torch.float64), t)
    with pytest.raises(RuntimeError, match="input tensor size must be equal to world_size times output tensor size"):
        pg._reduce_scatter_base(torch.empty(3), torch.empty(3 * world + 1))
    with pytest.raises(RuntimeError, match="number of output tensors should equal to the world size"):
        pg.allgather([[torch.empty(8)]], [t])
    with pytest.raises(RuntimeError, match="Tensors are not equal in data type"):
        pg.allgather([[torch.empty(8, dtype=torch.int32) for _ in range(world)]], [t])
    with pytest.raises(RuntimeError, match="does not divide equally across group size"):
        pg.alltoall_base(torch.empty(world + 1), torch.empty(world + 1), [], [])
    with pytest.raises(RuntimeError, match="number of input tensors are not equal to group size"):
        pg.alltoall([torch.empty(1)] * world, [torch.empty(1)] * (world + 1))
    with pytest.raises(RuntimeError, match="does not support recvAnysource"):
        pg.recv_anysource([t], 0)
    if rank != 0:
        g = dist.GatherOptions()
        g.rootRank = 0
        with pytest.raises(RuntimeError, match="number of output tensors should be 0 for non-root"):
            pg.gather([[torch.empty(8)] * world], [t], g)
    with pytest.raises(RuntimeError, match="Cannot use ReduceOp.BAND with non-integral dtype"):
        dist.all_reduce(t, op=dist.ReduceOp.BAND)
    dist.barrier()


def test_error_strings():
    run_ranks(_errors, world=2)


def _stress_and_coalescing(rank, world):
    # 1000 asynchronous broadcasts, all waited
    works = []
    ts = [torch.full((16,), float(i if rank == i % world else -1)) for i in range(1000)]
    for i, t in enumerate(ts):
        works.append(dist.broadcast(t, src=i % world, async_op=True))
    for w in works:
        w.wait()
    for i, t in enumerate(ts):
        assert torch.all(t == float(i))
    # coalescing manager: allreduce / all_gather_into_tensor / reduce_scatter_tensor
    from torch.distributed.distributed_c10d import _coalescing_manager

    a = [torch.full((10 + i,), float(rank + i)) for i in range(4)]
    with _coalescing_manager(device=torch.device("cpu"), async_ops=False):
        for t in a:
            dist.all_reduce(t)
    for i, t in enumerate(a):
        assert torch.all(t == sum(r + i for r in range(world)))
    ins = [torch.full((5,), float(rank * 10 + i)) for i in range(3)]
    outs = [torch.empty(5 * world) for _ in range(3)]
    with _coalescing_manager(device=torch.device("cpu"), async_ops=True) as cm:
        for o, i_ in zip(outs, ins):
            dist.all_gather_into_tensor(o, i_)
    cm.wait()
    for i, o in enumerate(outs):
        assert torch.equal(o, torch.cat([torch.full((5,), float(r * 10 + i)) for r in range(world)]))
    rs_in = [torch.arange(4.0 * world) + rank for _ in range(2)]
    rs_out = [torch.empty(4) for _ in range(2)]
    with _coalescing_manager(device=torch.device("cpu"), async_ops=False):
        for o, i_ in zip(rs_out, rs_in):
            dist.reduce_scatter_tensor(o, i_)
    ref = sum(torch.arange(4.0 * world) + r for r in range(world))
    for o in rs_out:
        assert torch.equal(o, ref[rank * 4:(rank + 1) * 4])
    # _broadcast_coalesced: the DDP initialisation path
    tensors = [torch.full((7,), float(rank)), torch.full((3, 3), float(rank) + 0.5)]
    dist._broadcast_coalesced(dist.group.WORLD, tensors, 256, 0)
    assert torch.all(tensors[0] == 0.0) and torch.all(tensors[1] == 0.5)
    # object collectives ride on the CPU path
    objs = [None] * world
    dist.all_gather_object(objs, {"rank": rank})
    assert [o["rank"] for o in objs] == list(range(world))
    # futures
    t = torch.ones(4)
    fut = dist.all_reduce(t, async_op=True).get_future()
    fut.wait()
    assert torch.all(fut.value()[0] == world)


def test_stress_coalescing_objects():
    run_ranks(_stress_and_coalescing, world=2)


def _ddp_and_subgroups(rank, world):
    torch.manual_seed(0)
    model = torch.nn.Linear(4, 5)
    ddp = torch.nn.parallel.DistributedDataParallel(model)
    x = torch.full((2, 4), float(rank + 1))
    for _ in range(3):
        ddp.zero_grad()
        ddp(x).sum().backward()
    ref = torch.stack([torch.full((4,), float(r + 1)) * 2 for r in range(world)]).mean(0)
    torch.testing.assert_close(model.weight.grad[0], ref)
    # singleton and strided sub-groups (cf. tests/ds_subgroup_allreduce.py:45-58 of the reference)
    solo = dist.new_group([0])
    if rank == 0:
        t = torch.ones(3)
        dist.all_reduce(t, group=solo)
        assert torch.all(t == 1)
    groups = [dist.new_group(list(range(s, world, 2))) for s in range(2)]
    mine = groups[rank % 2]
    t = torch.full((5,), float(rank), dtype=torch.bfloat16)
    dist.all_reduce(t, group=mine)
    assert torch.all(t == float(sum(range(rank % 2, world, 2))))
    dist.barrier()


def test_ddp_and_subgroups_world4():
    run_ranks(_ddp_and_subgroups, world=4)


def _two_virtual_nodes(rank, world):
    """Two 'nodes' of world/2 ranks each as separate communicators on one machine, plus the cross-node groups that pair
    equal local ranks: the hierarchical all_reduce (reduce_scatter inside the node, all_reduce across nodes, all_gather
    inside the node) must equal the flat one. This is the communicator layout a multi-node run would use."""
    per = world // 2
    node = rank // per
    local = rank % per
    node_groups = [dist.new_group(list(range(n * per, (n + 1) * per))) for n in range(2)]
    cross_groups = [dist.new_group([l, per + l]) for l in range(per)]
    intra, cross = node_groups[node], cross_groups[local]
    torch.manual_seed(7 + rank)
    x = torch.randn(per * 300)
    flat = x.clone()
    dist.all_reduce(flat)
    shard = torch.empty(300)
    dist.reduce_scatter_tensor(shard, x.clone(), group=intra)
    dist.all_reduce(shard, group=cross)
    out = torch.empty(per * 300)
    dist.all_gather_into_tensor(out, shard, group=intra)
    torch.testing.assert_close(out, flat, rtol=1e-5, atol=1e-5)
    # a broadcast that crosses the nodes first and fans out inside them afterwards
    b = torch.full((64,), float(rank))
    if local == 0:
        dist.broadcast(b, src=0, group=cross_groups[0])
    dist.broadcast(b, src=node * per, group=intra)
    assert torch.all(b == 0.0)
    dist.barrier()


def test_two_virtual_nodes_hierarchical_collectives():
    run_ranks(_two_virtual_nodes, world=4)


def _hierarchical_helper(rank, world, per):
    from torch_ccl_b200.parallel.hierarchical import HierarchicalGroups

    h = HierarchicalGroups(per)
    assert (h.nodes, h.node, h.local) == (world // per, rank // per, rank % per)
    torch.manual_seed(100 + rank)
    for n in (1, 7, 1000, 4099):  # not multiples of ranks_per_node: the helper pads
        x = torch.randn(n)
        flat = x.clone()
        dist.all_reduce(flat)
        h.all_reduce(x)
        torch.testing.assert_close(x, flat, rtol=1e-5, atol=1e-5)
    m = torch.randn(6, 10)
    want = m.t().contiguous()
    dist.all_reduce(want, op=dist.ReduceOp.MAX)
    view = m.t()  # non-contiguous
    h.all_reduce(view, op=dist.ReduceOp.MAX)
    assert torch.equal(view, want)
    for src in range(world):
        b = torch.full((33,), float(rank))
        h.broadcast(b, src)
        assert torch.all(b == float(src)), (src, b[0])
    piece = torch.arange(5.0) + 10 * rank
    got = torch.empty(5 * world)
    h.all_gather_into_tensor(got, piece)
    assert torch.equal(got, torch.cat([torch.arange(5.0) + 10 * r for r in range(world)]))
    full = torch.randn(world * 12)
    ref = full.clone()
    dist.all_reduce(ref)
    out = torch.empty(12)
    h.reduce_scatter_tensor(out, full)
    torch.testing.assert_close(out, ref[rank * 12:(rank + 1) * 12], rtol=1e-5, atol=1e-5)
    dist.barrier()


@pytest.mark.parametrize("per", [1, 2, 4])
def test_hierarchical_groups_match_flat_collectives(per):
    run_ranks(_hierarchical_helper, world=4, args=(per,))


def _p2p_patterns(rank, world):
    # relay 0 -> 1 -> 2 and all-pairs exchange with tags (accepted and ignored, like the reference)
    if rank == 0:
        dist.send(torch.arange(100.0), dst=1, tag=7)
    elif rank == 1:
        t = torch.empty(100)
        dist.recv(t, src=0, tag=7)
        dist.send(t * 2, dst=2, tag=9)
    elif rank == 2:
        t = torch.empty(100)
        dist.recv(t, src=1, tag=9)
        assert torch.equal(t, torch.arange(100.0) * 2)
    for a in range(world):
        for b in range(a + 1, world):
            if rank == a:
                dist.send(torch.full((10,), float(a * 10 + b)), dst=b)
            elif rank == b:
                t = torch.empty(10)
                dist.recv(t, src=a)
                assert torch.all(t == float(a * 10 + b))
    # ring exchange and the Ulysses layout change [s/N, h] -> [s, h/N] with all_to_all_single
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    r = torch.empty(4)
    reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, torch.full((4,), float(rank)), nxt), dist.P2POp(dist.irecv, r, prv)])
    for q in reqs:
        q.wait()
    assert torch.all(r == float(prv))
    s_local, heads = 3, 2 * world
    x = torch.arange(s_local * heads, dtype=torch.float32).view(s_local, heads) + 1000 * rank
    send = x.view(s_local, world, heads // world).transpose(0, 1).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send)
    full = torch.cat([torch.arange(s_local * heads, dtype=torch.float32).view(s_local, heads) + 1000 * p for p in range(world)])
    ref = full[:, rank * (heads // world):(rank + 1) * (heads // world)]
    assert torch.equal(recv.reshape(world * s_local, heads // world), ref)
    dist.barrier()


def test_p2p_relay_ring_ulysses_world3():
    run_ranks(_p2p_patterns, world=3)


def _profiler_ranges(rank, world):
    """Both levels of profiler ranges keep the reference's names (src/ProcessGroupCCL.cpp:995-1198
    `oneccl_bindings_for_pytorch::<op>` with the tensors as inputs, src/cpu/cpu_ccl.cpp:568,605
    `oneccl_bindings_for_pytorch::cpu::<op>`), so profiler scripts written against it keep working."""
    t = torch.ones(4, 4)
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU], record_shapes=True) as prof:
        dist.all_reduce(t)
        dist.broadcast(t, 0)
        outs = [torch.empty(4, 4) for _ in range(world)]
        dist.all_gather(outs, t)
        dist.barrier()
    keys = {e.key: e for e in prof.key_averages(group_by_input_shape=True)}
    names = {k for k in (e.key for e in prof.key_averages())}
    for op in ("allreduce", "broadcast", "allgather", "barrier"):
        assert "oneccl_bindings_for_pytorch::" + op in names, sorted(names)
    for op in ("allreduce", "broadcast", "allgather"):
        assert "oneccl_bindings_for_pytorch::cpu::" + op in names, sorted(names)
    shaped = [e for e in prof.key_averages(group_by_input_shape=True) if e.key == "oneccl_bindings_for_pytorch::allreduce"]
    assert shaped and any([4, 4] in e.input_shapes for e in shaped), [e.input_shapes for e in shaped]
    del keys


def test_profiler_ranges_world2():
    run_ranks(_profiler_ranges, world=2)


def test_bench_reference_arm_reports_unavailable():
    """`bench.py --impl reference` must answer on any machine: the reference (a binding over Intel oneCCL + SYCL for
    Intel GPUs) cannot be installed here, so the arm prints one JSON line saying so and exits 0."""
    import json
    import subprocess
    import sys

    from mp_util import ROOT

    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line.get("unavailable"), str) and line["unavailable"]
