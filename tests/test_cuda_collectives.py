"""The c10d surface on CUDA tensors with one process per GPU (needs >= 2 GPUs): every collective
against plain torch math, Work semantics, DDP, sub-groups and NCCL-backed send/recv."""
import os

import pytest
import torch
import torch.distributed as dist

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

SIZES = [1, 7, 4096, 458752 + 1, (8 << 20) + 3]


def _world():
    return min(torch.cuda.device_count(), int(os.environ.get("CCL_TEST_WORLD", "8")))


def _data(rank, n, dtype=torch.float32, salt=0):
    g = torch.Generator().manual_seed(99 + 31 * rank + salt)
    return torch.randn(n, generator=g, dtype=torch.float64).to(dtype)


def _tol(dtype, world):
    t = {torch.bfloat16: 2e-2, torch.float16: 4e-3, torch.float32: 1e-5}[dtype]
    return dict(rtol=t, atol=t * world)


def _allreduce(rank, world):
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for n in SIZES:
            xs = [_data(r, n, dtype) for r in range(world)]
            ref = torch.stack([x.double() for x in xs]).sum(0)
            t = xs[rank].cuda()
            dist.all_reduce(t)
            torch.testing.assert_close(t.cpu().double(), ref.to(dtype).double(), **_tol(dtype, world))
            # all ranks hold bitwise the same result
            gathered = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(gathered, t)
            for g in gathered:
                assert torch.equal(g, gathered[0])
    x = _data(rank, 1000).cuda()
    ref = torch.stack([_data(r, 1000) for r in range(world)])
    for op, r in [(dist.ReduceOp.AVG, ref.mean(0)), (dist.ReduceOp.MAX, ref.max(0).values), (dist.ReduceOp.MIN, ref.min(0).values)]:
        t = x.clone()
        dist.all_reduce(t, op=op)
        torch.testing.assert_close(t.cpu(), r, rtol=1e-5, atol=1e-5)
    ti = torch.arange(100, device="cuda", dtype=torch.int64) + rank
    dist.all_reduce(ti, op=dist.ReduceOp.BXOR)
    r = torch.zeros(100, dtype=torch.int64)
    for k in range(world):
        r ^= torch.arange(100) + k
    assert torch.equal(ti.cpu(), r)
    # async op + wait, coalesced
    ts = [torch.full((50,), float(rank + i), device="cuda") for i in range(3)]
    work = dist.all_reduce_coalesced(ts, async_op=True) if hasattr(dist, "all_reduce_coalesced") else None
    if work is not None:
        work.wait()
        for i, t in enumerate(ts):
            assert torch.all(t == sum(range(world)) + world * i)


def _coalesced(rank, world):
    """The *_coalesced entry points: a list of small tensors goes out as ONE kernel launch (pointer table)."""
    import torch_ccl_b200

    be = dist.group.WORLD._get_backend(torch.device("cuda"))
    sizes = [3, 1000, 17, 40000]
    ts = [torch.full((n,), float(rank + i), device="cuda") for i, n in enumerate(sizes)]
    n0 = be.cuda_kernel_launches(ts[0])
    dist.all_reduce_coalesced(ts)
    torch.cuda.synchronize()
    assert be.cuda_kernel_launches(ts[0]) == n0 + 1, "one launch for the whole list"
    for i, t in enumerate(ts):
        assert torch.all(t == sum(range(world)) + world * i)
    assert "multi" in torch_ccl_b200.flight_recorder()
    ins = [_data(rank, n, torch.bfloat16, salt=i).cuda() for i, n in enumerate(sizes)]
    outs = [torch.empty(n * world, dtype=torch.bfloat16, device="cuda") for n in sizes]
    n0 = be.cuda_kernel_launches(ts[0])
    dist.group.WORLD.allgather_into_tensor_coalesced(outs, ins).wait()
    torch.cuda.synchronize()
    assert be.cuda_kernel_launches(ts[0]) == n0 + 1
    for i, n in enumerate(sizes):
        assert torch.equal(outs[i].cpu(), torch.cat([_data(r, n, torch.bfloat16, salt=i) for r in range(world)]))
    full = [_data(rank, n * world, salt=10 + i).cuda() for i, n in enumerate(sizes)]
    parts = [torch.empty(n, device="cuda") for n in sizes]
    n0 = be.cuda_kernel_launches(ts[0])
    dist.group.WORLD.reduce_scatter_tensor_coalesced(parts, full).wait()
    torch.cuda.synchronize()
    assert be.cuda_kernel_launches(ts[0]) == n0 + 1
    for i, n in enumerate(sizes):
        ref = torch.stack([_data(r, n * world, salt=10 + i) for r in range(world)]).sum(0)[rank * n:(rank + 1) * n]
        torch.testing.assert_close(parts[i].cpu(), ref, rtol=1e-5, atol=1e-5)
    dist.barrier()


def _rooted(rank, world):
    n = 300001
    xs = [_data(r, n) for r in range(world)]
    for root in {0, world - 1}:
        t = xs[rank].cuda()
        dist.reduce(t, dst=root)
        if rank == root:
            torch.testing.assert_close(t.cpu(), torch.stack(xs).sum(0), rtol=1e-5, atol=1e-5)
        t = xs[rank].cuda()
        dist.broadcast(t, src=root)
        assert torch.equal(t.cpu(), xs[root])
        g = [torch.empty(n, device="cuda") for _ in range(world)] if rank == root else None
        dist.gather(xs[rank].cuda(), g, dst=root)
        if rank == root:
            for r in range(world):
                assert torch.equal(g[r].cpu(), xs[r])
        out = torch.empty(n, device="cuda")
        dist.scatter(out, [x.cuda() for x in xs] if rank == root else None, src=root)
        assert torch.equal(out.cpu(), xs[rank])
    with pytest.raises(ValueError, match="unexpected rank"):
        dist.group.WORLD._get_backend(torch.device("cuda")).broadcast([torch.zeros(1, device="cuda")], _bad_opts(world))


def _bad_opts(world):
    o = dist.BroadcastOptions()
    o.rootRank = world
    return o


def _gather_scatter_family(rank, world):
    for n in (1, 4099, 1 << 20):
        xs = [_data(r, n, torch.bfloat16) for r in range(world)]
        outs = [torch.empty(n, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        dist.all_gather(outs, xs[rank].cuda())
        for r in range(world):
            assert torch.equal(outs[r].cpu(), xs[r])
        flat = torch.empty(world * n, dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(flat, xs[rank].cuda())
        assert torch.equal(flat.cpu(), torch.cat(xs))
        full = [_data(r, n * world, salt=3) for r in range(world)]
        out = torch.empty(n, device="cuda")
        dist.reduce_scatter_tensor(out, full[rank].cuda())
        ref = torch.stack(full).sum(0)[rank * n:(rank + 1) * n]
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-5)
    # uneven reduce_scatter list
    cnt = [3 + 100 * p for p in range(world)]
    ins = [[_data(r, cnt[p], salt=p) for p in range(world)] for r in range(world)]
    out = torch.empty(cnt[rank], device="cuda")
    dist.reduce_scatter(out, [t.cuda() for t in ins[rank]])
    torch.testing.assert_close(out.cpu(), sum(ins[r][rank] for r in range(world)), rtol=1e-5, atol=1e-5)
    # all_to_all: equal, uneven single, list
    x = _data(rank, world * 1000).cuda()
    o = torch.empty_like(x)
    dist.all_to_all_single(o, x)
    ref = torch.cat([_data(r, world * 1000)[rank * 1000:(rank + 1) * 1000] for r in range(world)])
    assert torch.equal(o.cpu(), ref)
    send = [[1 + ((r * 7 + p * 3) % 5) * 1000 for p in range(world)] for r in range(world)]
    xin = _data(rank, sum(send[rank]), salt=5).cuda()
    recv = [send[p][rank] for p in range(world)]
    o = torch.empty(sum(recv), device="cuda")
    dist.all_to_all_single(o, xin, output_split_sizes=recv, input_split_sizes=send[rank])
    pieces = []
    for p in range(world):
        off = sum(send[p][:rank])
        pieces.append(_data(p, sum(send[p]), salt=5)[off:off + send[p][rank]])
    assert torch.equal(o.cpu(), torch.cat(pieces))
    dist.barrier()


def _work_semantics_and_ddp(rank, world):
    t = torch.ones(1 << 20, device="cuda")
    w = dist.all_reduce(t, async_op=True)
    w.wait()
    assert float(t[0]) == world
    fut = dist.all_reduce(t, async_op=True).get_future()
    fut.wait()
    assert float(t[-1]) == world * world
    # DDP over the backend: gradients are averaged across ranks
    torch.manual_seed(0)
    model = torch.nn.Linear(64, 32).cuda()
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[torch.cuda.current_device()])
    x = _data(rank, 16 * 64).view(16, 64).cuda()
    ddp(x).sum().backward()
    g = model.weight.grad.clone()
    ref = torch.stack([_data(r, 16 * 64).view(16, 64).sum(0) for r in range(world)]).mean(0)
    torch.testing.assert_close(g[0].cpu(), ref, rtol=1e-4, atol=1e-4)
    # sub-group of the even ranks
    even = list(range(0, world, 2))
    sub = dist.new_group(even)
    if rank in even:
        s = torch.full((1000,), float(rank), device="cuda")
        dist.all_reduce(s, group=sub)
        assert float(s[0]) == sum(even)
    dist.barrier()


def _p2p(rank, world):
    if rank == 0:
        dist.send(torch.arange(1000.0, device="cuda"), dst=1)
    elif rank == 1:
        t = torch.empty(1000, device="cuda")
        dist.recv(t, src=0)
        assert torch.equal(t.cpu(), torch.arange(1000.0))
    # ring exchange with batched isend/irecv
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    s = torch.full((4096,), float(rank), device="cuda")
    r = torch.empty(4096, device="cuda")
    reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, s, nxt), dist.P2POp(dist.irecv, r, prv)])
    for q in reqs:
        q.wait()
    torch.cuda.synchronize()
    assert torch.all(r == float(prv))
    dist.barrier()


@pytest.mark.parametrize("fn", [_allreduce, _coalesced, _rooted, _gather_scatter_family, _work_semantics_and_ddp, _p2p],
                         ids=lambda f: f.__name__.strip("_"))
def test_cuda_ranks(fn):
    run_ranks(fn, world=_world(), device="cuda", env={"NCCL_NVLS_ENABLE": "0", "CCL_ARENA_MB": "64"}, timeout=300)


def _blocking_same_stream(rank, world):
    t = torch.ones(100000, device="cuda")
    for _ in range(10):
        dist.all_reduce(t)
        t /= world
    torch.cuda.synchronize()
    assert torch.allclose(t, torch.ones_like(t))


@pytest.mark.parametrize("env", [{"CCL_BLOCKING_WAIT": "1"}, {"CCL_SAME_STREAM": "1"}, {"TORCH_LLM_ALLREDUCE": "1"}],
                         ids=["blocking_wait", "same_stream", "llm_allreduce"])
def test_cuda_modes(env):
    e = {"NCCL_NVLS_ENABLE": "0", "CCL_ARENA_MB": "64"}
    e.update(env)
    run_ranks(_blocking_same_stream, world=_world(), device="cuda", env=e, timeout=300)


def _fused_gemm_ops(rank, world):
    from torch_ccl_b200 import ops

    torch.manual_seed(11)
    M, N, Kl = world * 256, 512, 256
    As = [torch.randn(M, Kl, generator=torch.Generator().manual_seed(r)).to(torch.bfloat16) for r in range(world)]
    Bs = [(torch.randn(N, Kl, generator=torch.Generator().manual_seed(100 + r)) * 0.1).to(torch.bfloat16) for r in range(world)]
    for _ in range(3):
        out = ops.gemm_reduce_scatter(As[rank].cuda(), Bs[rank].cuda())
    torch.cuda.synchronize()
    ref = sum((As[r].float() @ Bs[r].float().t()).to(torch.bfloat16).float() for r in range(world))
    rows = M // world
    torch.testing.assert_close(out.cpu().float(), ref[rank * rows:(rank + 1) * rows], rtol=2e-2, atol=0.2)
    shard = [torch.randn(128, 320, generator=torch.Generator().manual_seed(200 + r)).to(torch.bfloat16) for r in range(world)]
    w = (torch.randn(256, 320, generator=torch.Generator().manual_seed(300 + rank)) * 0.1).to(torch.bfloat16)
    for _ in range(3):
        out2 = ops.all_gather_gemm(shard[rank].cuda(), w.cuda())
    torch.cuda.synchronize()
    torch.testing.assert_close(out2.cpu().float(), torch.cat(shard).float() @ w.float().t(), rtol=2e-2, atol=0.2)
    t = torch.ones(10, device="cuda")
    dist.all_reduce(t)
    assert float(t[0]) == world
    dist.barrier()


def test_cuda_fused_gemm_collectives():
    run_ranks(_fused_gemm_ops, world=_world(), device="cuda", env={"NCCL_NVLS_ENABLE": "0", "CCL_ARENA_MB": "64"}, timeout=300)


def _fsdp_engine(rank, world):
    """The fused full-shard engine must train exactly like the same schedule on plain c10d calls."""
    import torch.nn as nn

    from torch_ccl_b200.parallel.fsdp import FullyShardedSequential

    def make():
        torch.manual_seed(0)
        return [nn.Sequential(nn.Linear(64, 96), nn.GELU()).cuda(), nn.Linear(96, 64).cuda(), nn.Linear(64, 8).cuda()]

    losses = {}
    for comm in ("c10d", "ccl_symmetric", "ccl"):
        # "ccl_symmetric": parameter / gradient buffers from the symmetric heap, zero-copy collectives
        eng = FullyShardedSequential(make(), comm="ccl" if comm.startswith("ccl") else comm, symmetric=comm == "ccl_symmetric",
                                     comm_blocks=16 if comm == "ccl_symmetric" else None)
        opt = torch.optim.SGD(eng.master_params(), lr=0.02)
        out = []
        for it in range(3):
            x = _data(rank, 16 * 64).view(16, 64).cuda().to(torch.bfloat16)  # same batch every step: the loss must fall
            loss = eng(x).float().pow(2).mean()
            loss.backward()
            eng.master_params()
            opt.step()
            eng.after_step()
            out.append(float(loss))
        losses[comm] = out
    for arm in ("ccl", "ccl_symmetric"):
        for a, b in zip(losses[arm], losses["c10d"]):
            assert abs(a - b) <= 2e-2 * max(1.0, abs(b)), (losses)
    assert losses["ccl"][-1] < losses["ccl"][0]
    # sharded checkpoint: save, perturb, reload -> the same loss; consolidated copy on rank 0
    import io

    buf = io.BytesIO()
    torch.save(eng.sharded_state_dict(), buf)
    x = _data(rank, 16 * 64).view(16, 64).cuda().to(torch.bfloat16)
    with torch.no_grad():
        before = float(eng(x).float().pow(2).mean())
        for u in eng.units:
            u.master.add_(1.0)
            u.sync_shard()
        eng.after_step()
        assert abs(float(eng(x).float().pow(2).mean()) - before) > 1e-3
        buf.seek(0)
        eng.load_sharded_state_dict(torch.load(buf))
        assert float(eng(x).float().pow(2).mean()) == before
    full = eng.full_state_dict(0)
    if rank == 0:
        assert full["0.0.weight"].shape == (96, 64) and full["2.bias"].shape == (8,) and len(full) == 6
    else:
        assert full is None
    with pytest.raises(ValueError, match="does not fit"):
        eng.load_sharded_state_dict({"world": world + 1, "rank": rank, "units": []})
    dist.barrier()


def test_cuda_fsdp_engine_and_moe_ops():
    run_ranks(_fsdp_engine, world=_world(), device="cuda", env={"NCCL_NVLS_ENABLE": "0", "CCL_ARENA_MB": "64", "CCL_SPIN_TIMEOUT_MS": "3000",
                                                                   "CCL_SYMM_HEAP_MB": "64", "CCL_SYMM_MIN_BYTES": "0"}, timeout=180)


def _tp_decode(rank, world):
    """Tensor-parallel decode on real peers: the fused step (projection + all_reduce + residual + norm in one
    kernel, fused sampling) against the fp32 restatement over plain all_reduces, eager and from a CUDA graph,
    and against the unfused kernels."""
    from torch_ccl_b200.models.llama import LlamaConfig, TPLlamaDecoder

    cfg = LlamaConfig(vocab=1024, hidden=512, n_layers=2, n_heads=8, n_kv_heads=8, inter=1408 if world != 8 else 2048)
    B = 4
    m = TPLlamaDecoder(cfg, max_batch=B, max_seq=256, seed=3)
    u = TPLlamaDecoder(cfg, max_batch=B, max_seq=256, seed=3, fused=False)
    assert m.fused and not u.fused
    prompt = torch.randint(0, cfg.vocab, (B, 40), generator=torch.Generator().manual_seed(5))
    m.prefill(prompt)
    u.prefill(prompt)
    assert torch.equal(m.tokens, u.tokens)
    for step in range(3):
        u.tokens.copy_(m.tokens)
        ref = m.reference_decode_step(B)
        m.decode_step(B)
        u.decode_step(B)
        torch.cuda.synchronize()
        torch.testing.assert_close(m.logits[:B], ref, rtol=3e-2, atol=3e-2)
        # same rounding points, but the split-K factor (and so the fp32 summation order) may differ
        torch.testing.assert_close(m.logits[:B], u.logits[:B], rtol=2e-2, atol=2e-2)
    e = TPLlamaDecoder(cfg, max_batch=B, max_seq=256, seed=3)
    e.prefill(prompt)
    for L1, L2 in zip(e.layers, m.layers):  # bring the eager twin to the same state as m
        L1["k"].copy_(L2["k"])
        L1["v"].copy_(L2["v"])
    e.tokens.copy_(m.tokens)
    e.positions.copy_(m.positions)
    m.capture(B)
    for step in range(4):
        a = m.decode_step(B).clone()
        b = e.decode_step(B).clone()
        assert torch.equal(a, b), "graph replay and eager launches of the fused step must agree bit for bit"
    assert int(m.positions[0]) == 40 + 7
    # every rank holds the same sampled ids
    g = [torch.empty_like(a) for _ in range(world)]
    dist.all_gather(g, a)
    for t in g:
        assert torch.equal(t, g[0])
    be = dist.group.WORLD._get_backend(torch.device("cuda"))
    assert be.cuda_comm_status(a)[0] == 0
    dist.barrier()


def test_cuda_tp_decode_fused():
    run_ranks(_tp_decode, world=_world(), device="cuda", env={"NCCL_NVLS_ENABLE": "0", "CCL_ARENA_MB": "64", "CCL_SPIN_TIMEOUT_MS": "5000"}, timeout=300)


def _streams_and_coalescing(rank, world):
    """Ordering across streams: a coalescing window of CUDA collectives issued from a side stream must order that
    stream after them, and a fused op on the caller's stream must not overlap a c10d op still in flight on the
    backend's communication stream (both use the same communicator state)."""
    from torch.distributed.distributed_c10d import _coalescing_manager

    from torch_ccl_b200 import ops

    side = torch.cuda.Stream()
    n = 1 << 20
    for it in range(5):
        with torch.cuda.stream(side):
            a = torch.full((n,), float(rank + it), device="cuda")
            b = torch.full((n,), float(rank), device="cuda")
            with _coalescing_manager(device=torch.device("cuda"), async_ops=True) as cm:
                dist.all_reduce(a)
                dist.broadcast(b, src=world - 1)
            cm.wait()
            # consumers on the side stream: must see the finished collectives
            sa, sb = a.sum(), b.sum()
        side.synchronize()
        assert float(sa) == float(n) * (sum(range(world)) + world * it), (float(sa), it)
        assert float(sb) == float(n) * (world - 1)
    # async c10d op followed at once by a fused op on the current stream
    for it in range(5):
        big = torch.ones(4 << 20, device="cuda")
        w = dist.all_reduce(big, async_op=True)
        small = torch.full((1000,), 2.0, device="cuda")
        ops.all_reduce_scaled(small, 0.5)
        w.wait()
        torch.cuda.synchronize()
        assert float(big[-1]) == world and float(small[0]) == world
    be = dist.group.WORLD._get_backend(torch.device("cuda"))
    assert be.cuda_comm_status(big)[0] == 0
    dist.barrier()


def test_cuda_streams_and_coalescing():
    run_ranks(_streams_and_coalescing, world=_world(), device="cuda", env={"NCCL_NVLS_ENABLE": "0", "CCL_ARENA_MB": "64", "CCL_SPIN_TIMEOUT_MS": "5000"}, timeout=300)


def test_kernels_configure_each_device():
    """One process, two GPUs: the shared-memory opt-in of a kernel is a per-device attribute, so the GEMM, the
    attention and the allocation-free attention entry point must work on device 1 after they ran on device 0."""
    import ctypes
    import glob

    import torch_ccl_b200._C as C
    from torch_ccl_b200.ops import gemm_bf16_tn

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = ctypes.CDLL(glob.glob(os.path.join(root, "torch_ccl_b200", "_C*.so"))[0])
    fn = lib.ccl_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong] + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    results = []
    for d in (0, 1):
        with torch.cuda.device(d):
            dev = torch.device("cuda", d)
            g = torch.Generator(device=dev).manual_seed(1)
            a = torch.randn(256, 4096, device=dev, generator=g).to(torch.bfloat16)
            b = torch.randn(16, 4096, device=dev, generator=g).to(torch.bfloat16)
            out = gemm_bf16_tn(a, b, trans_out=True, splitk=4, bn=16)       # > 48 KB of dynamic shared memory
            big = gemm_bf16_tn(torch.randn(4096, 512, device=dev, generator=g).to(torch.bfloat16),
                               torch.randn(4096, 512, device=dev, generator=g).to(torch.bfloat16))  # persistent kernel
            torch.testing.assert_close(out.float(), b.float() @ a.float().t(), rtol=2e-2, atol=2.0)
            B, nh, nkv, hd, S, ns = 2, 4, 2, 128, 512, 3
            qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=dev, generator=g).to(torch.bfloat16)
            kc = torch.randn(B, nkv, S, hd, device=dev, generator=g).to(torch.bfloat16)
            vc = torch.randn(B, nkv, S, hd, device=dev, generator=g).to(torch.bfloat16)
            pos = torch.tensor([100, 400], device=dev, dtype=torch.int32)
            tab = torch.zeros(S, hd // 2, device=dev)
            o1 = torch.empty(B, nh * hd, device=dev, dtype=torch.bfloat16)
            o2 = torch.empty_like(o1)
            scratch = torch.zeros(C.decode_attention_scratch_bytes(B, nh, ns) // 4 + 1, device=dev)
            counters = torch.zeros(B * nh, device=dev, dtype=torch.int32)
            k1, v1 = kc.clone(), vc.clone()
            C.decode_attention(qkv, k1, v1, pos, tab + 1.0, tab, o1, scratch, counters, nh, nkv, ns)
            k2, v2 = kc.clone(), vc.clone()
            cos = tab + 1.0
            rc = fn(qkv.data_ptr(), qkv.stride(0), k2.data_ptr(), v2.data_ptr(), pos.data_ptr(), cos.data_ptr(), tab.data_ptr(),
                    o2.data_ptr(), o2.stride(0), B, nh, nkv, hd, S, ns, torch.cuda.current_stream(dev).cuda_stream)
            assert rc == 0, lib.ccl_noalloc_last_error()
            torch.cuda.synchronize(dev)
            torch.testing.assert_close(o1.float(), o2.float(), rtol=2e-2, atol=2e-2)
            results.append((out.float().cpu(), o1.float().cpu(), big.float().cpu()))
    for x, y in zip(results[0], results[1]):
        torch.testing.assert_close(x, y, rtol=2e-2, atol=2.0)
