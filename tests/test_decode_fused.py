"""The decode-step kernels that fold a collective into the kernel next to it, on ONE GPU: a single
launch with gridDim.y == world plays every rank of the communicator.

  * gemm_ar_norm: row-parallel projection + all_reduce + residual add + RMSNorm in one launch
  * the embedding lookup fused in front of the all_reduce + norm kernel
  * sample_allgather: arg-max over vocabulary shards + all-gather of the winners

Oracles are plain PyTorch fp32 restatements with the rounding points of the unfused sequence."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def comms():
    import torch_ccl_b200._C as C

    made = []

    def make(world, half=1 << 20):
        c = C.CudaComm.emulated(world, half, 2000, 8)
        made.append(c)
        return c

    yield make
    torch.cuda.synchronize()
    made.clear()


def _norm_ref(partials, res, w, eps):
    s = torch.stack([p.float() for p in partials]).sum(0).to(torch.bfloat16)
    h = (s.float() + res.float()).to(torch.bfloat16)
    hf = h.float()
    n = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16)
    return h, (n.float() * w.float()).to(torch.bfloat16)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("rows,hidden,k,splitk", [
    (16, 512, 192, 0), (1, 512, 64, 1), (4, 512, 200, 2), (16, 1024, 512, 4), (16, 512, 1376, 8),
    (24, 512, 320, 0), (40, 512, 256, 4), (13, 768, 136, 8)])
def test_gemm_ar_norm(comms, world, rows, hidden, k, splitk):
    from torch_ccl_b200.ops import pack_weight

    c = comms(world)
    assert c.fits_gemm_ar_norm(rows, hidden, k)
    torch.manual_seed(world * 1000 + rows + k)
    ws = [(torch.randn(hidden, k) * 0.05).to(torch.bfloat16) for _ in range(world)]
    wn = (torch.rand(hidden) + 0.5).to(torch.bfloat16)
    res0 = torch.randn(rows, hidden).to(torch.bfloat16)
    dws = [pack_weight(w.cuda()) for w in ws]
    dwn = [wn.cuda() for _ in range(world)]
    dres = [res0.clone().cuda() for _ in range(world)]
    douts = [torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    h_ref = res0
    for it in range(3):  # repeated calls: epoch, parity and the residual stream keep in step
        xs = [torch.randn(rows, k).to(torch.bfloat16) for _ in range(world)]
        dxs = [x.cuda() for x in xs]
        c.gemm_ar_norm(dws, dxs, dres, dwn, douts, 1e-5, splitk)
        torch.cuda.synchronize()
        assert c.status()[0] == 0, c.status()
        partials = [(x.float() @ w.float().t()).to(torch.bfloat16) for x, w in zip(xs, ws)]
        h_ref, o_ref = _norm_ref(partials, h_ref, wn, 1e-5)
        for r in range(world):
            torch.testing.assert_close(dres[r].cpu().float(), h_ref.float(), rtol=2e-2, atol=8e-2)
            torch.testing.assert_close(douts[r].cpu().float(), o_ref.float(), rtol=2e-2, atol=8e-2)
        for r in range(1, world):
            assert torch.equal(douts[r], douts[0]) and torch.equal(dres[r], dres[0])
        h_ref = dres[0].cpu()  # follow the kernel's residual stream so that rounding does not accumulate in the oracle


def test_gemm_ar_norm_equals_unfused_sequence(comms):
    """Bit-identical to GEMM -> all_reduce -> add -> rmsnorm done by the separate kernels."""
    import torch_ccl_b200._C as C
    from torch_ccl_b200.ops import pack_weight

    world, rows, hidden, k = 4, 16, 1024, 384
    c = comms(world)
    torch.manual_seed(7)
    ws = [pack_weight((torch.randn(hidden, k) * 0.05).to(torch.bfloat16).cuda()) for _ in range(world)]
    xs = [torch.randn(rows, k).to(torch.bfloat16).cuda() for _ in range(world)]
    wn = [(torch.rand(hidden) + 0.5).to(torch.bfloat16).cuda() for _ in range(world)]
    res = torch.randn(rows, hidden).to(torch.bfloat16)
    r1 = [res.clone().cuda() for _ in range(world)]
    r2 = [res.clone().cuda() for _ in range(world)]
    o1 = [torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    o2 = [torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    c.gemm_ar_norm(ws, xs, r1, wn, o1, 1e-5, 4)
    parts = []
    for r in range(world):
        p = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
        C.gemm_bf16_tn(ws[r], xs[r], p, True, 0, 4, 16, hidden)
        parts.append(p)
    c.allreduce_residual_rmsnorm(parts, r2, wn, o2, 1e-5)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    for r in range(world):
        assert torch.equal(o1[r], o2[r]) and torch.equal(r1[r], r2[r])


@pytest.mark.parametrize("world", [1, 2, 8])
def test_embedding_lookup_fused_into_allreduce_norm(comms, world):
    c = comms(world)
    vocab, hidden, rows = 64 * world, 512, 9
    vs = vocab // world
    torch.manual_seed(3)
    table = torch.randn(vocab, hidden).to(torch.bfloat16)
    wn = (torch.rand(hidden) + 0.5).to(torch.bfloat16)
    toks = torch.randint(0, vocab, (rows,))
    shards = [table[r * vs:(r + 1) * vs].contiguous().cuda() for r in range(world)]
    dres = [torch.full((rows, hidden), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]  # must be ignored
    douts = [torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for _ in range(2):
        c.allreduce_residual_rmsnorm(shards, dres, [wn.cuda()] * world, douts, 1e-5, [toks.cuda()] * world,
                                     [r * vs for r in range(world)], True)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    h = table[toks]
    hf = h.float()
    n = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16)
    o = (n.float() * wn.float()).to(torch.bfloat16)
    for r in range(world):
        assert torch.equal(dres[r].cpu(), h)
        torch.testing.assert_close(douts[r].cpu().float(), o.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_sample_allgather(comms, world):
    c = comms(world)
    rows, vs = 16, 1000
    torch.manual_seed(11)
    logits = torch.randn(rows, vs * world)
    logits[3, 17] = logits[3, vs * (world - 1) + 25] = 9.0  # a tie (across the first and the last shard): lowest id wins
    shards = [logits[:, r * vs:(r + 1) * vs].contiguous().cuda() for r in range(world)]
    nxt = [torch.zeros(rows, dtype=torch.int64, device="cuda") for _ in range(world)]
    tok = [torch.zeros(rows, dtype=torch.int64, device="cuda") for _ in range(world)]
    pos = [torch.arange(rows, dtype=torch.int32, device="cuda") for _ in range(world)]
    for it in range(3):
        c.sample_allgather(shards, nxt, tok, pos)
    torch.cuda.synchronize()
    assert c.status()[0] == 0
    ref = logits.argmax(dim=-1)
    assert int(ref[3]) == 17
    for r in range(world):
        assert torch.equal(nxt[r].cpu(), ref) and torch.equal(tok[r].cpu(), ref)
        assert torch.equal(pos[r].cpu(), torch.arange(rows, dtype=torch.int32) + 3)


def test_abort_word_ends_a_wait_early():
    """abort(): a kernel that waits for a peer that never arrives returns as soon as the host raises the
    communicator's abort word, long before its wait budget, and reports the aborted status."""
    import time

    import torch_ccl_b200._C as C

    c = C.CudaComm.emulated(2, 1 << 20, 3000, 1)  # 3 s budget: only the abort can end the wait sooner
    t0 = time.time()
    assert C.emu_missing_peer_probe(c)  # plays rank 0 of a barrier only: waits on a flag nothing sets
    time.sleep(0.05)
    c.abort()
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.5
    st = c.status()
    assert st[0] == 3 and st[2] == 1, st  # kStatusAborted, waited for rank 1
    c.clear_abort()
    x = torch.ones(8, device="cuda")
    assert float((x + 1).sum()) == 16.0  # context alive
