"""Numerics of the tcgen05 bf16 GEMM against a plain fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    import torch_ccl_b200._C as C

    return C


def _ref(a, b):
    return a.float() @ b.float().t()


def _check(out, ref, k):
    tol = 2e-2 * (k ** 0.5) * 0.05 + 1e-2
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= 1e-2 * scale + tol * 0.1, f"max err {err} (scale {scale})"


@pytest.mark.parametrize("M,N,K,bn", [
    (128, 16, 64, 16), (128, 16, 256, 16), (256, 128, 512, 128), (300, 72, 328, 0),
    (1024, 256, 4096, 256), (512, 64, 1024, 64), (128, 32, 2048, 32),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_plain(M, N, K, bn, out_dtype):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=out_dtype)
    _C().gemm_bf16_tn(a, b, out, False, 0, 1, bn)
    torch.cuda.synchronize()
    _check(out, _ref(a, b), K)


@pytest.mark.parametrize("batch", [1, 4, 16])
@pytest.mark.parametrize("splitk", [1, 2, 4, 8, 16, 0])
def test_gemm_swap_ab_splitk(batch, splitk):
    """Decode shape: weights on the UMMA M side, the few activation rows on the N side."""
    torch.manual_seed(1)
    n_out, K = 1536, 4096
    w = torch.randn(n_out, K, device="cuda", dtype=torch.bfloat16) * 0.05
    x = torch.randn(batch, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(batch, n_out, device="cuda", dtype=torch.bfloat16)
    _C().gemm_bf16_tn(w, x, out, True, 0, splitk, 16)
    torch.cuda.synchronize()
    _check(out, _ref(x, w), K)


@pytest.mark.parametrize("splitk", [1, 2, 4, 16])
def test_gemm_dual_swiglu(splitk):
    torch.manual_seed(2)
    inter, K, batch = 1376, 4096, 16
    w = torch.randn(2 * inter, K, device="cuda", dtype=torch.bfloat16) * 0.03
    x = torch.randn(batch, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(batch, inter, device="cuda", dtype=torch.bfloat16)
    _C().gemm_bf16_tn(w, x, out, True, inter, splitk, 16)
    torch.cuda.synchronize()
    g = x.float() @ w[:inter].float().t()
    u = x.float() @ w[inter:].float().t()
    ref = torch.nn.functional.silu(g) * u
    _check(out, ref, K)


@pytest.mark.parametrize("M,N,K,bn", [(2048, 2560, 512, 128), (4096, 2560, 320, 256), (2000, 2500, 328, 128),
                                      (3000, 3100, 1032, 256), (8192, 4096, 4096, 0)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_persistent(M, N, K, bn, out_dtype):
    """>= 148 tiles and no split-K: the persistent kernel with double-buffered TMEM accumulators."""
    torch.manual_seed(3)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=out_dtype)
    _C().gemm_bf16_tn(a, b, out, False, 0, 1, bn)
    torch.cuda.synchronize()
    _check(out, _ref(a, b), K)


@pytest.mark.parametrize("rows,K,batch", [(1536, 4096, 16), (1000, 1376, 5), (4096, 512, 16), (4096, 1376, 130)])
@pytest.mark.parametrize("splitk", [0, 1, 3, 16])
def test_gemm_pretiled_weights(rows, K, batch, splitk):
    """Weights packed as contiguous 128x64 tiles (ops.pack_weight), rows / K padded with zeros."""
    from torch_ccl_b200.ops import pack_weight, unpack_weight

    torch.manual_seed(4)
    w = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16) * 0.05
    x = torch.randn(batch, K, device="cuda", dtype=torch.bfloat16)
    packed = pack_weight(w)
    assert torch.equal(unpack_weight(packed, rows, K), w)
    out = torch.empty(batch, rows, device="cuda", dtype=torch.bfloat16)
    bn = 16 if batch <= 16 else 128
    _C().gemm_bf16_tn(packed, x, out, True, 0, 1 if bn == 128 else splitk, bn, rows)
    torch.cuda.synchronize()
    _check(out, _ref(x, w), K)


@pytest.mark.parametrize("batch", [16, 200])
def test_gemm_pretiled_swiglu(batch):
    from torch_ccl_b200.ops import pack_weight

    torch.manual_seed(5)
    inter, K = 1376, 4096
    wg = torch.randn(inter, K, device="cuda", dtype=torch.bfloat16) * 0.03
    wu = torch.randn(inter, K, device="cuda", dtype=torch.bfloat16) * 0.03
    x = torch.randn(batch, K, device="cuda", dtype=torch.bfloat16)
    packed = torch.cat([pack_weight(wg), pack_weight(wu)])
    pad = (inter + 127) // 128 * 128
    out = torch.empty(batch, inter, device="cuda", dtype=torch.bfloat16)
    bn = 16 if batch <= 16 else 128
    _C().gemm_bf16_tn(packed, x, out, True, pad, 0 if bn == 16 else 1, bn, inter)
    torch.cuda.synchronize()
    ref = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    _check(out, ref, K)
