"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of this library get raw device pointers and a stream and are not allowed to allocate
device memory (a custom op inside an inference server that owns the memory pool, a call made
while a graph capture is in progress elsewhere on the device, a process confined to a fixed memory
slice). For them `ccl_decode_attention_noalloc` keeps the split-KV scratch inside the library.
This test loads the built extension with ctypes, calls the symbol twice in a row on the same
inputs and checks both results against the regular entry point (which takes a caller-provided
scratch buffer), within the tolerance of the other attention tests; it also checks that a request
beyond the built-in scratch is refused with a clear message. The file name sorts last so that
every other test has already run if this one fails."""
import ctypes
import glob
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    import torch_ccl_b200._C as C  # noqa: F401  (makes sure torch's libraries are loaded first)

    path = glob.glob(os.path.join(ROOT, "torch_ccl_b200", "_C*.so"))[0]
    lib = ctypes.CDLL(path)
    fn = lib.ccl_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.ccl_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _attention_fp32(qkv, kc, vc, pos, cos, sin, nh, nkv):
    """Plain PyTorch fp32 restatement: rotate q and k of the new token, attend over cache[:pos] plus the new k/v."""
    B, hd = qkv.shape[0], 128
    outs = []
    for b in range(B):
        p = int(pos[b])
        c, s = cos[p], sin[p]

        def rope(t):
            t1, t2 = t[..., :64], t[..., 64:]
            return torch.cat([t1 * c - t2 * s, t2 * c + t1 * s], -1)

        q = rope(qkv[b, : nh * hd].float().view(nh, hd))
        k = rope(qkv[b, nh * hd:(nh + nkv) * hd].float().view(nkv, hd)).to(torch.bfloat16)
        v = qkv[b, (nh + nkv) * hd:].view(nkv, hd)
        kk = torch.cat([kc[b, :, :p], k[:, None]], 1).float().repeat_interleave(nh // nkv, 0)
        vv = torch.cat([vc[b, :, :p], v[:, None]], 1).float().repeat_interleave(nh // nkv, 0)
        sc = torch.einsum("hd,htd->ht", q, kk) / hd ** 0.5
        outs.append(torch.einsum("ht,htd->hd", sc.softmax(-1), vv).reshape(-1))
    return torch.stack(outs)


def test_noalloc_entry_matches_regular_entry_twice():
    import torch_ccl_b200._C as C

    lib, fn = _lib()
    torch.manual_seed(0)
    B, nh, nkv, hd, S, nsplit = 3, 8, 4, 128, 700, 5
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
    kc = torch.randn(B, nkv, S, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(B, nkv, S, hd, device="cuda", dtype=torch.bfloat16)
    pos = torch.tensor([5, 333, 698], device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()

    # regular entry point: caller-provided scratch
    k_ref, v_ref = kc.clone(), vc.clone()
    ref = torch.empty(B, nh * hd, device="cuda", dtype=torch.bfloat16)
    scratch = torch.zeros(C.decode_attention_scratch_bytes(B, nh, nsplit) // 4 + 1, device="cuda")
    counters = torch.zeros(B * nh, device="cuda", dtype=torch.int32)
    C.decode_attention(qkv, k_ref, v_ref, pos, cos, sin, ref, scratch, counters, nh, nkv, nsplit)
    torch.cuda.synchronize()

    stream = torch.cuda.current_stream().cuda_stream
    before = torch.cuda.memory_allocated()
    for call in range(2):
        k2, v2 = kc.clone(), vc.clone()
        out = torch.zeros(B, nh * hd, device="cuda", dtype=torch.bfloat16)
        base = torch.cuda.memory_allocated()
        rc = fn(qkv.data_ptr(), qkv.stride(0), k2.data_ptr(), v2.data_ptr(), pos.data_ptr(), cos.data_ptr(),
                sin.data_ptr(), out.data_ptr(), out.stride(0), B, nh, nkv, hd, S, nsplit, stream)
        assert rc == 0, lib.ccl_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == base, "the entry point must not allocate through torch"
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out.float(), _attention_fp32(qkv, kc, vc, pos, cos, sin, nh, nkv), rtol=2e-2, atol=2e-2)
        assert torch.equal(k2, k_ref) and torch.equal(v2, v_ref), f"KV append differs on call {call}"
    assert torch.cuda.memory_allocated() >= before


def test_noalloc_entry_rejects_oversized_requests():
    lib, fn = _lib()
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    rc = fn(p, 0, p, p, p, p, p, p, 0, 64, 32, 32, 128, 1024, 4, 0)  # 64*32*4 = 8192 > 4096 partials
    assert rc == 1
    msg = lib.ccl_noalloc_last_error().decode()
    assert "exceeds the built-in scratch" in msg and "8192" in msg
    assert fn(p, 0, p, p, p, p, p, p, 0, 1, 8, 4, 64, 128, 1, 0) == 2  # unsupported head_dim


def test_noalloc_entry_rejects_bad_layouts_without_launching():
    """A misaligned pointer or a row stride that is short or not a multiple of 8 elements would fault the
    16-byte accesses of the kernel: the entry point returns 2 and launches nothing."""
    lib, fn = _lib()
    B, nh, nkv, hd, S = 2, 4, 2, 128, 256
    width = (nh + 2 * nkv) * hd
    qkv = torch.zeros(B, width + 8, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(B, nkv, S, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    pos = torch.zeros(B, device="cuda", dtype=torch.int32)
    tab = torch.zeros(S, hd // 2, device="cuda")
    out = torch.full((B, nh * hd + 8), 3.0, device="cuda", dtype=torch.bfloat16)

    def call(q_ptr, q_stride, o_ptr, o_stride):
        return fn(q_ptr, q_stride, kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), tab.data_ptr(), tab.data_ptr(), o_ptr, o_stride,
                  B, nh, nkv, hd, S, 1, torch.cuda.current_stream().cuda_stream)

    assert call(qkv.data_ptr() + 2, qkv.stride(0), out.data_ptr(), out.stride(0)) == 2      # qkv not 16-byte aligned
    assert "aligned" in lib.ccl_noalloc_last_error().decode()
    assert call(qkv.data_ptr(), width + 4, out.data_ptr(), out.stride(0)) == 2              # stride not a multiple of 8
    assert call(qkv.data_ptr(), width - 8, out.data_ptr(), out.stride(0)) == 2              # rows would overlap
    assert call(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), nh * hd - 8) == 2            # out rows would overlap
    torch.cuda.synchronize()
    assert bool((out == 3.0).all()), "nothing may have been launched"
    assert call(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0)) == 0          # the well-formed call goes through
    torch.cuda.synchronize()


def test_out_of_range_position_is_contained():
    """A position outside the cache gives a zero row and leaves the cache alone instead of indexing out of bounds."""
    lib, fn = _lib()
    B, nh, nkv, hd, S = 2, 4, 2, 128, 256
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
    kc = torch.randn(B, nkv, S, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    k0 = kc.clone()
    pos = torch.tensor([S + 5, 10], device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    out = torch.full((B, nh * hd), 3.0, device="cuda", dtype=torch.bfloat16)
    rc = fn(qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(),
            out.data_ptr(), out.stride(0), B, nh, nkv, hd, S, 2, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert bool((out[0] == 0).all()) and torch.equal(kc[0], k0[0])
    assert bool(out[1].float().abs().sum() > 0)
