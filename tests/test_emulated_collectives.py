"""Every peer-memory collective kernel, run as ONE cooperative launch that plays all ranks on a
single GPU (gridDim.y = world), checked against plain PyTorch math on the same inputs.

Oracle: the mathematical definition evaluated in fp64 on the CPU and rounded to the tensor dtype
(the reference's own LLM all-reduce test compares a SUM to its input and cannot serve:
tests/test_llm_allreduce.py:40-46 of intel/torch-ccl).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

SUM, PROD, MIN, MAX, BAND, BOR, BXOR = range(7)
SIZES = [1, 7, 8, 1000, 4096, 65537]
WORLDS = [2, 3, 8]


@pytest.fixture(scope="module")
def comms():
    import torch_ccl_b200._C as C

    cache = {}

    def get(world, half_bytes=8 << 20):
        key = (world, half_bytes)
        if key not in cache:
            cache[key] = C.CudaComm.emulated(world, half_bytes, 2000, 8)
        return cache[key]

    yield get
    cache.clear()


def rand(n, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    if dtype.is_floating_point:
        return torch.randn(n, generator=g, dtype=torch.float64).to(dtype)
    return torch.randint(-50, 50, (n,), generator=g, dtype=torch.int64).to(dtype)


def oracle_reduce(xs, op, dtype):
    stack = torch.stack([x.double() if dtype.is_floating_point else x.long() for x in xs])
    if op == SUM:
        r = stack.sum(0)
    elif op == PROD:
        r = stack.prod(0)
    elif op == MIN:
        r = stack.min(0).values
    elif op == MAX:
        r = stack.max(0).values
    else:
        r = stack[0]
        for s in stack[1:]:
            r = {BAND: r & s, BOR: r | s, BXOR: r ^ s}[op]
    return r


def close(out, ref, dtype, world):
    if dtype.is_floating_point:
        tol = {torch.bfloat16: 2e-2, torch.float16: 4e-3, torch.float32: 1e-5, torch.float64: 1e-12}[dtype]
        torch.testing.assert_close(out.cpu().double(), ref.double().to(dtype).double(), rtol=tol, atol=tol * world)
    else:
        assert torch.equal(out.cpu().long(), ref.to(dtype).long())


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("algo", [1, 2])
def test_allreduce_sum(comms, world, n, dtype, algo):
    c = comms(world)
    xs = [rand(n, dtype, 100 + r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    outs = [torch.empty_like(t) for t in ins]
    for _ in range(3):  # repeated calls exercise the epoch / parity protocol
        c.allreduce(ins, outs, SUM, 1.0, 0, algo)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    ref = oracle_reduce(xs, SUM, dtype)
    for o in outs:
        close(o, ref, dtype, world)
    for o in outs[1:]:
        assert torch.equal(o, outs[0]), "ranks must agree bitwise"


@pytest.mark.parametrize("dtype,op", [
    (torch.float16, MAX), (torch.float64, PROD), (torch.int32, BXOR), (torch.int64, MIN),
    (torch.uint8, BOR), (torch.int8, SUM), (torch.int16, BAND),
])
@pytest.mark.parametrize("algo", [1, 2])
def test_allreduce_ops_dtypes(comms, dtype, op, algo):
    world, n = 4, 3001
    c = comms(world)
    if dtype == torch.uint8:
        xs = [torch.randint(0, 255, (n,), generator=torch.Generator().manual_seed(r), dtype=torch.int64).to(dtype) for r in range(world)]
    elif op == PROD:
        xs = [(rand(n, dtype, r) * 0.5 + 1.0) for r in range(world)]
    else:
        xs = [rand(n, dtype, 7 + r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    c.allreduce(ins, ins, op, 1.0, 0, algo)  # in place
    torch.cuda.synchronize()
    ref = oracle_reduce(xs, op, dtype)
    for o in ins:
        close(o, ref, dtype, world)


def test_allreduce_avg_and_unaligned(comms):
    world, n = 8, 5003
    c = comms(world)
    xs = [rand(n + 1, torch.bfloat16, r) for r in range(world)]
    bufs = [x.cuda() for x in xs]
    ins = [b[1:] for b in bufs]  # 2-byte aligned views
    outs = [torch.empty(n + 1, dtype=torch.bfloat16, device="cuda")[1:] for _ in range(world)]
    for algo in (1, 2):
        c.allreduce(ins, outs, SUM, 1.0 / world, 1, algo)
        torch.cuda.synchronize()
        ref = oracle_reduce([x[1:] for x in xs], SUM, torch.bfloat16) / world
        for o in outs:
            close(o, ref, torch.bfloat16, world)


def test_allreduce_multi_round(comms):
    """A message larger than the arena: several staging rounds inside one launch."""
    world = 4
    c = comms(world, 1 << 20)
    n = (3 << 20) // 4 + 13
    xs = [rand(n, torch.float32, r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    tag = c.allreduce(ins, ins, SUM, 1.0, 0, 0)
    torch.cuda.synchronize()
    assert tag.startswith("twoshot")
    ref = oracle_reduce(xs, SUM, torch.float32)
    for o in ins:
        close(o, ref, torch.float32, world)


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("root", [0, 1])
def test_reduce_to_root(comms, world, root):
    c = comms(world)
    n = 10007
    xs = [rand(n, torch.float32, 50 + r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    outs = [torch.full_like(t, -7.0) for t in ins]
    c.reduce(ins, outs, SUM, root)
    c.reduce(ins, outs, SUM, root)
    torch.cuda.synchronize()
    close(outs[root], oracle_reduce(xs, SUM, torch.float32), torch.float32, world)
    for r in range(world):
        if r != root:
            assert torch.all(outs[r] == -7.0), "non-root outputs must stay untouched"


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("n", [1, 9, 4096, 30001])
def test_reduce_scatter_equal(comms, world, n):
    c = comms(world)
    xs = [rand(n * world, torch.float32, r) for r in range(world)]
    flat = [x.cuda() for x in xs]
    ins = [[f[p * n:(p + 1) * n] for p in range(world)] for f in flat]
    outs = [torch.empty(n, device="cuda") for _ in range(world)]
    for _ in range(2):
        c.reduce_scatter(ins, outs, SUM, 1.0, 0)
    torch.cuda.synchronize()
    ref = oracle_reduce(xs, SUM, torch.float32)
    for r in range(world):
        close(outs[r], ref[r * n:(r + 1) * n], torch.float32, world)


def test_reduce_scatter_uneven_and_fused_cast(comms):
    """Pieces of different sizes; bf16 gradients averaged and written as fp32 in one pass."""
    world = 4
    c = comms(world)
    cnt = [5, 4096, 0, 777]
    xs = [[rand(cnt[p], torch.bfloat16, 10 * r + p) for p in range(world)] for r in range(world)]
    ins = [[t.cuda() for t in row] for row in xs]
    outs = [torch.empty(cnt[r], device="cuda", dtype=torch.float32) for r in range(world)]
    c.reduce_scatter(ins, outs, SUM, 1.0 / world, 1)
    torch.cuda.synchronize()
    for r in range(world):
        ref = torch.stack([xs[s][r].double() for s in range(world)]).sum(0) / world
        torch.testing.assert_close(outs[r].cpu().double(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("n", [1, 33, 70000, 300000])
def test_all_gather(comms, world, n):
    c = comms(world)
    xs = [rand(n, torch.bfloat16, r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    flat = [torch.empty(n * world, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    outs = [[f[p * n:(p + 1) * n] for p in range(world)] for f in flat]
    for _ in range(2):
        c.all_gather(ins, outs)
    torch.cuda.synchronize()
    ref = torch.cat(xs)
    for f in flat:
        assert torch.equal(f.cpu(), ref)


def test_all_gather_uneven(comms):
    world = 3
    c = comms(world)
    cnt = [3, 0, 1025]
    xs = [rand(cnt[r], torch.int32, r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    outs = [[torch.empty(cnt[p], dtype=torch.int32, device="cuda") for p in range(world)] for _ in range(world)]
    c.all_gather(ins, outs)
    torch.cuda.synchronize()
    for r in range(world):
        for p in range(world):
            assert torch.equal(outs[r][p].cpu(), xs[p])


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("uneven", [False, True])
def test_all_to_all(comms, world, uneven):
    c = comms(world, 1 << 20)
    g = torch.Generator().manual_seed(3)
    if uneven:
        cnt = torch.randint(0, 40000, (world, world), generator=g).tolist()
        cnt[0][world - 1] = 0
    else:
        cnt = [[20011] * world for _ in range(world)]
    xs = [[rand(cnt[r][p], torch.float32, 100 * r + p) for p in range(world)] for r in range(world)]
    ins = [[t.cuda() for t in row] for row in xs]
    outs = [[torch.empty(cnt[p][r], device="cuda") for p in range(world)] for r in range(world)]
    for _ in range(2):
        c.all_to_all(ins, outs, uneven)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    for r in range(world):
        for p in range(world):
            assert torch.equal(outs[r][p].cpu(), xs[p][r])


def test_all_to_all_uneven_multi_round(comms):
    """Uneven pieces larger than a staging slot: ranks agree on the round count on the device."""
    world = 2
    c = comms(world, 1 << 20)
    cnt = [[10, 400000], [5, 70]]
    xs = [[rand(cnt[r][p], torch.float32, 100 * r + p) for p in range(world)] for r in range(world)]
    ins = [[t.cuda() for t in row] for row in xs]
    outs = [[torch.empty(cnt[p][r], device="cuda") for p in range(world)] for r in range(world)]
    c.all_to_all(ins, outs, True)
    torch.cuda.synchronize()
    for r in range(world):
        for p in range(world):
            assert torch.equal(outs[r][p].cpu(), xs[p][r])


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("root", [0, 1])
def test_broadcast_gather_scatter(comms, world, root):
    c = comms(world, 1 << 20)
    n = 300001  # > one staging round for gather
    xs = [rand(n, torch.float32, 9 + r) for r in range(world)]
    bufs = [x.cuda() for x in xs]
    for _ in range(2):
        c.broadcast(bufs, root)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b.cpu(), xs[root])
    ins = [x.cuda() for x in xs]
    gathered = [torch.empty(n, device="cuda") for _ in range(world)]
    c.gather(ins, gathered, root)
    torch.cuda.synchronize()
    for p in range(world):
        assert torch.equal(gathered[p].cpu(), xs[p])
    outs = [torch.empty(n, device="cuda") for _ in range(world)]
    c.scatter(ins, outs, root)
    torch.cuda.synchronize()
    for p in range(world):
        assert torch.equal(outs[p].cpu(), xs[p])


def test_barrier_and_mixed_sequence(comms):
    world = 8
    c = comms(world)
    xs = [rand(999, torch.float32, r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    ref = oracle_reduce(xs, SUM, torch.float32)
    for i in range(20):
        c.barrier()
        outs = [torch.empty_like(t) for t in ins]
        c.allreduce(ins, outs, SUM, 1.0, 0, 1 + (i % 2))
        bufs = [t.clone() for t in ins]
        c.broadcast(bufs, i % world)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    close(outs[0], ref, torch.float32, world)


def _rmsnorm_ref(xs, res, w, eps, dtype):
    s = torch.stack([x.float() for x in xs]).sum(0).to(dtype)
    h = (s.float() + res.float()).to(dtype)
    hf = h.float()
    n = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)
    return h, (n.float() * w.float()).to(dtype)


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("rows", [1, 4, 16, 40])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_allreduce_residual_rmsnorm(comms, world, rows, dtype):
    hidden = 4096
    c = comms(world)
    torch.manual_seed(0)
    xs = [torch.randn(rows, hidden).to(dtype) for _ in range(world)]
    res = torch.randn(rows, hidden).to(dtype)
    w = (torch.rand(hidden) + 0.5).to(dtype)
    dx = [x.cuda() for x in xs]
    dres = [res.clone().cuda() for _ in range(world)]
    dw = [w.cuda() for _ in range(world)]
    douts = [torch.empty(rows, hidden, dtype=dtype, device="cuda") for _ in range(world)]
    c.allreduce_residual_rmsnorm(dx, dres, dw, douts, 1e-5)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    h_ref, o_ref = _rmsnorm_ref(xs, res, w, 1e-5, dtype)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    for r in range(world):
        torch.testing.assert_close(dres[r].cpu().float(), h_ref.float(), rtol=tol, atol=tol * 4)
        torch.testing.assert_close(douts[r].cpu().float(), o_ref.float(), rtol=tol, atol=tol * 4)
    for r in range(1, world):
        assert torch.equal(douts[r], douts[0])


def test_bounded_wait_reports_timeout_instead_of_hanging():
    """A rank that never shows up: the waiting kernel gives up after its budget, records who it
    waited for, and returns; the context stays usable. Emulated by a world-2 communicator whose
    launch only plays rank 0 (nctx trick is not available, so the sync-only ablation of a
    one-rank launch is used: the wait is on a flag nobody sets)."""
    import torch_ccl_b200._C as C

    c = C.CudaComm.emulated(2, 1 << 20, 200, 1)
    ok = C.emu_missing_peer_probe(c)
    torch.cuda.synchronize()
    st = c.status()
    assert ok and st[0] == 1, st  # kStatusTimeout
    assert st[2] == 1  # peer that never signalled
    x = torch.ones(8, device="cuda")
    assert float((x + 1).sum()) == 16.0  # context alive


@pytest.mark.parametrize("world", [2, 4])
def test_gemm_reduce_scatter_fused(comms, world):
    """Row-parallel linear + reduce-scatter in one pass: tcgen05 tiles pushed into the owners'
    arenas from the epilogue, then summed. Oracle: fp32 matmul of the concatenated K shards."""
    c = comms(world, 8 << 20)
    torch.manual_seed(5)
    M, N, Kl = world * 256, 384, 320
    As = [torch.randn(M, Kl).to(torch.bfloat16) for _ in range(world)]
    Bs = [(torch.randn(N, Kl) * 0.1).to(torch.bfloat16) for _ in range(world)]
    outs = [torch.empty(M // world, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    da, db = [a.cuda() for a in As], [b.cuda() for b in Bs]
    for _ in range(3):  # repeated calls: counters, epochs and parity keep in step
        c.gemm_rs(da, db, outs)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    parts = [As[r].float() @ Bs[r].float().t() for r in range(world)]
    ref = sum(p.to(torch.bfloat16).float() for p in parts)  # partials travel as bf16
    rows = M // world
    for r in range(world):
        torch.testing.assert_close(outs[r].cpu().float(), ref[r * rows:(r + 1) * rows], rtol=2e-2, atol=0.15)


@pytest.mark.parametrize("world", [2, 4])
def test_all_gather_gemm_fused(comms, world):
    """All-gather + column-parallel linear: shards pushed into the peers' arenas, tiles of a
    shard start as soon as its arrival counter is reached."""
    c = comms(world, 8 << 20)
    torch.manual_seed(6)
    rows, K, Nl = 128, 448, 272
    As = [torch.randn(rows, K).to(torch.bfloat16) for _ in range(world)]
    Bs = [(torch.randn(Nl, K) * 0.1).to(torch.bfloat16) for _ in range(world)]
    outs = [torch.empty(world * rows, Nl, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    da, db = [a.cuda() for a in As], [b.cuda() for b in Bs]
    for _ in range(3):
        c.ag_gemm(da, db, outs)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    full = torch.cat(As).float()
    for r in range(world):
        torch.testing.assert_close(outs[r].cpu().float(), full @ Bs[r].float().t(), rtol=2e-2, atol=0.15)
    # an op of the ordinary kind right after: the shared epoch must still line up
    xs = [torch.full((1000,), float(r + 1), device="cuda") for r in range(world)]
    c.allreduce(xs, xs, SUM, 1.0, 0, 1)
    torch.cuda.synchronize()
    assert float(xs[0][0]) == sum(range(1, world + 1))


@pytest.mark.parametrize("world,epr", [(2, 1), (4, 2), (8, 1)])
def test_moe_dispatch_combine(comms, world, epr):
    """Fused expert-parallel exchange: tokens routed top-2 to experts spread over the ranks. The
    dispatch must deliver exactly the routed rows (any order) with correct records; after an
    'expert' that scales each row by (1 + local expert id), combine must equal the dense formula."""
    c = comms(world, 8 << 20)
    T, K, H = 96, 2, 256
    E = world * epr
    g = torch.Generator().manual_seed(21)
    xs = [torch.randn(T, H, generator=g).to(torch.bfloat16) for _ in range(world)]
    idx = [torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32) for _ in range(world)]
    gate = [torch.rand(T, K, generator=g) for _ in range(world)]
    cap_rows = world * T * K
    dx = [x.cuda() for x in xs]
    di = [i.cuda() for i in idx]
    out_x = [torch.zeros(cap_rows, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    meta = [torch.zeros(cap_rows, 3, dtype=torch.int32, device="cuda") for _ in range(world)]
    count = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(world)]
    outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for rep in range(2):
        c.moe_dispatch(dx, di, out_x, meta, count, epr)
        torch.cuda.synchronize()
        assert c.status()[0] == 0
        ys = []
        for r in range(world):
            n = int(count[r][0])
            expect = sum(int(((idx[s] // epr) == r).sum()) for s in range(world))
            assert n == expect
            m = meta[r][:n].cpu()
            rows = out_x[r][:n].cpu()
            for i in range(0, n, max(1, n // 17)):
                s, slot, le = m[i].tolist()
                assert torch.equal(rows[i], xs[s][slot // K])
                assert int(idx[s].view(-1)[slot]) == r * epr + le
            y = out_x[r].clone()
            y[:n] = (rows.float() * (1.0 + m[:, 2:3].float())).to(torch.bfloat16).cuda()
            ys.append(y)
        c.moe_combine(ys, meta, count, [gt.cuda() for gt in gate], outs)
        torch.cuda.synchronize()
        assert c.status()[0] == 0
        for r in range(world):
            le = (idx[r] % epr).float()
            scaled = torch.stack([(xs[r].float() * (1.0 + le[:, k:k + 1])).to(torch.bfloat16).float() for k in range(K)], 1)
            ref = (scaled * gate[r][:, :, None]).sum(1)
            torch.testing.assert_close(outs[r].cpu().float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n", [1, 1000, 65537])
def test_allreduce_switch_reduction_emulated(comms, world, dtype, n):
    """The multicast (NVLS) all_reduce kernel with its two multimem operations played in software:
    checks staging layout, shard ownership, flag pairing and copy-out for every world size."""
    c = comms(world)
    xs = [rand(n, dtype, 300 + r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    outs = [torch.empty_like(t) for t in ins]
    for _ in range(3):
        tag = c.allreduce(ins, outs, SUM, 1.0, 0, 3)
    torch.cuda.synchronize()
    assert tag.startswith("nvls") and c.status()[0] == 0
    ref = oracle_reduce(xs, SUM, dtype)
    for o in outs:
        close(o, ref, dtype, world)
    for o in outs[1:]:
        assert torch.equal(o, outs[0]), "ranks must agree bitwise"


def test_allreduce_switch_reduction_multi_round_scale_and_fallback(comms):
    world = 4
    c = comms(world, 1 << 20)
    n = (3 << 20) // 4 + 13  # 3 MB through 1 MB halves: several rounds
    xs = [rand(n, torch.float32, r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    tag = c.allreduce(ins, ins, SUM, 1.0 / world, 1, 3)  # in place, averaged
    torch.cuda.synchronize()
    assert tag.startswith("nvls")
    ref = oracle_reduce(xs, SUM, torch.float32) / world
    for o in ins:
        close(o, ref, torch.float32, world)
    # the switch only adds: MAX falls back to the peer-memory kernels
    ys = [rand(1000, torch.float32, 50 + r).cuda() for r in range(world)]
    tag = c.allreduce(ys, ys, MAX, 1.0, 0, 3)
    assert not tag.startswith("nvls")


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_reduce_scatter_switch_reduction_emulated(comms, world, dtype):
    c = comms(world)
    cnt = [1000 + 37 * p for p in range(world)]  # uneven pieces
    xs = [[rand(cnt[p], dtype, 10 * r + p) for p in range(world)] for r in range(world)]
    ins = [[t.cuda() for t in row] for row in xs]
    outs = [torch.empty(cnt[r], dtype=dtype, device="cuda") for r in range(world)]
    for _ in range(2):
        c.reduce_scatter(ins, outs, SUM, 1.0, 0, True)
    torch.cuda.synchronize()
    assert c.last_used_nvls and c.status()[0] == 0
    for r in range(world):
        close(outs[r], oracle_reduce([xs[q][r] for q in range(world)], SUM, dtype), dtype, world)
    # the widened gradient path (bf16 in, fp32 out) keeps the peer-load kernel
    if dtype == torch.bfloat16:
        wide = [torch.empty(cnt[r], dtype=torch.float32, device="cuda") for r in range(world)]
        c.reduce_scatter(ins, wide, SUM, 1.0, 0, True)
        assert not c.last_used_nvls


@pytest.mark.parametrize("world,root", [(2, 1), (3, 0), (8, 5)])
def test_broadcast_switch_multicast_emulated(comms, world, root):
    """Broadcast whose root stores every vector once into the multicast address (played in software here), mixed with
    the peer-store broadcast and an all_reduce so that the arena halves and epochs of consecutive kernels interleave."""
    c = comms(world, 1 << 20)
    n = 700001  # 2.8 MB of float32 through 1 MB halves: three rounds, ragged tail
    xs = [rand(n, torch.float32, 40 + r) for r in range(world)]
    bufs = [x.cuda() for x in xs]
    c.broadcast(bufs, root, True)
    torch.cuda.synchronize()
    assert c.last_used_nvls and c.status()[0] == 0
    for b in bufs:
        assert torch.equal(b.cpu(), xs[root])
    ys = [rand(1000, torch.float32, 90 + r).cuda() for r in range(world)]
    other = (root + 1) % world
    bytes8 = [rand(4099, torch.float32, 60 + r).view(torch.uint8)[:16385].clone() for r in range(world)]  # odd byte count
    b8 = [t.cuda() for t in bytes8]
    for _ in range(2):
        c.allreduce(ys, ys, SUM, 1.0, 0, 0)
        c.broadcast(b8, other, True)
        c.broadcast(bufs, other, False)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    for b in b8:
        assert torch.equal(b.cpu(), bytes8[other])
    for b in bufs:
        assert torch.equal(b.cpu(), xs[root])  # every buffer already held the root's data


@pytest.mark.parametrize("world", [2, 3, 8])
def test_all_gather_switch_multicast_emulated(comms, world):
    c = comms(world, 1 << 20)
    cnt = [70001 + 13 * p for p in range(world)]  # uneven, several rounds through 1 MB halves at world 8
    xs = [rand(cnt[r], torch.float32, 77 + r) for r in range(world)]
    ins = [x.cuda() for x in xs]
    outs = [[torch.empty(cnt[p], device="cuda") for p in range(world)] for _ in range(world)]
    for _ in range(2):
        c.all_gather(ins, outs, True)
    torch.cuda.synchronize()
    assert c.last_used_nvls and c.status()[0] == 0
    for r in range(world):
        for p in range(world):
            assert torch.equal(outs[r][p].cpu(), xs[p])
