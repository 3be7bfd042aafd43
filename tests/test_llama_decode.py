"""The tensor-parallel Llama decoder on one GPU (world 1): the kernel path (tcgen05 GEMMs, fused
RoPE/KV-append/split-KV attention, fused add+RMSNorm, CUDA graph) against a plain PyTorch fp32
restatement of the same step, and prefill against token-by-token decoding."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(batch=4, max_seq=512, layers=2):
    from torch_ccl_b200.models.llama import LlamaConfig, TPLlamaDecoder

    return TPLlamaDecoder(LlamaConfig.tiny(layers), max_batch=batch, max_seq=max_seq, seed=3)


def test_decode_attention_matches_reference():
    import torch_ccl_b200._C as C

    torch.manual_seed(0)
    B, nh, nkv, hd, S = 3, 8, 4, 128, 700
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
    kc = torch.randn(B, nkv, S, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(B, nkv, S, hd, device="cuda", dtype=torch.bfloat16)
    pos = torch.tensor([0, 333, 698], device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    for nsplit in (1, 3, 8):
        k2, v2 = kc.clone(), vc.clone()
        out = torch.empty(B, nh * hd, device="cuda", dtype=torch.bfloat16)
        scratch = torch.zeros(C.decode_attention_scratch_bytes(B, nh, nsplit) // 4 + 1, device="cuda")
        counters = torch.zeros(B * nh, device="cuda", dtype=torch.int32)
        for _ in range(2):  # second launch checks that the counters were re-armed
            C.decode_attention(qkv, k2, v2, pos, cos, sin, out, scratch, counters, nh, nkv, nsplit)
        torch.cuda.synchronize()
        for b in range(B):
            p = int(pos[b])
            c, s = cos[p], sin[p]

            def rope(t):
                t1, t2 = t[..., :64], t[..., 64:]
                return torch.cat([t1 * c - t2 * s, t2 * c + t1 * s], -1)

            q = rope(qkv[b, : nh * hd].float().view(nh, hd))
            k = rope(qkv[b, nh * hd:(nh + nkv) * hd].float().view(nkv, hd)).to(torch.bfloat16)
            v = qkv[b, (nh + nkv) * hd:].view(nkv, hd)
            assert torch.equal(k2[b, :, p], k) and torch.equal(v2[b, :, p], v), "KV append"
            kk = torch.cat([kc[b, :, :p], k[:, None]], 1).float().repeat_interleave(nh // nkv, 0)
            vv = torch.cat([vc[b, :, :p], v[:, None]], 1).float().repeat_interleave(nh // nkv, 0)
            sc = torch.einsum("hd,htd->ht", q, kk) / hd ** 0.5
            ref = torch.einsum("ht,htd->hd", sc.softmax(-1), vv).reshape(-1)
            torch.testing.assert_close(out[b].float(), ref, rtol=2e-2, atol=2e-2)


def test_decode_step_matches_reference():
    m = _model()
    B = 4
    torch.manual_seed(1)
    m.tokens[:B] = torch.randint(0, m.cfg.vocab, (B,), device="cuda")
    for step in range(5):
        ref = m.reference_decode_step(B)
        m.decode_step(B)
        torch.cuda.synchronize()
        got = m.logits[:B]
        torch.testing.assert_close(got, ref, rtol=3e-2, atol=3e-2)
        assert int(m.positions[0]) == step + 1
        m.tokens[:B] = m.next_tokens[:B]


def test_graph_replay_equals_eager():
    m1, m2 = _model(), _model()
    B = 4
    toks = torch.randint(0, m1.cfg.vocab, (B,), device="cuda")
    m1.tokens[:B] = toks
    m2.tokens[:B] = toks
    m2.capture(B)
    assert int(m2.positions[0]) == 0
    for _ in range(4):
        a = m1.decode_step(B).clone()
        b = m2.decode_step(B).clone()
        assert torch.equal(a, b)
    pin_in = torch.zeros(B, dtype=torch.int64).pin_memory()
    pin_out = torch.zeros(B, dtype=torch.int64).pin_memory()
    pin_in.copy_(m1.next_tokens[:B].cpu())
    ref = m1.decode_step(B).cpu()
    out = m2.decode_step_host(pin_in, pin_out)
    assert torch.equal(out, ref)


def test_prefill_matches_token_by_token():
    m1, m2 = _model(batch=2), _model(batch=2)
    S = 130
    prompt = torch.randint(0, m1.cfg.vocab, (2, S))
    m1.prefill(prompt)
    for t in range(S):
        m2.tokens[:2] = prompt[:, t].cuda()
        m2.decode_step(2)
    torch.cuda.synchronize()
    assert int(m1.positions[0]) == S and int(m2.positions[0]) == S
    for L1, L2 in zip(m1.layers, m2.layers):
        torch.testing.assert_close(L1["k"][:, :, :S].float(), L2["k"][:, :, :S].float(), rtol=5e-2, atol=5e-2)
        torch.testing.assert_close(L1["v"][:, :, :S].float(), L2["v"][:, :, :S].float(), rtol=5e-2, atol=5e-2)
