"""Sequence-parallel tensor-parallel layers (torch_ccl_b200.parallel.tensor_parallel) against a dense
single-process layer: forward values, input gradients and weight gradients, on CPU ranks; the
CUDA variant additionally takes the fused GEMM + collective forward path when the shapes allow."""
import math

import pytest
import torch
import torch.distributed as dist

from mp_util import run_ranks


def _full_weight(out_f, in_f, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.empty(out_f, in_f).uniform_(-1.0, 1.0, generator=g) / math.sqrt(in_f)


def _tp_mlp(rank, world, device, S, hidden, inner, dtype_name, tol):
    from torch_ccl_b200.parallel.tensor_parallel import ParallelMLP

    dtype = getattr(torch, dtype_name)
    dev = torch.device("cuda", torch.cuda.current_device()) if device == "cuda" else torch.device("cpu")
    g = torch.Generator().manual_seed(5)
    x_full = torch.randn(S, hidden, generator=g)
    gy_full = torch.randn(S, hidden, generator=g)
    rows = S // world
    x = x_full[rank * rows:(rank + 1) * rows].to(dev, dtype).requires_grad_(True)
    mlp = ParallelMLP(hidden, inner, seed=11, device=dev, dtype=dtype)
    y = mlp(x)
    assert y.shape == (rows, hidden)
    y.backward(gy_full[rank * rows:(rank + 1) * rows].to(dev, dtype))

    # dense reference in fp64 on the full sequence
    w_up = _full_weight(inner, hidden, 11).double().requires_grad_(True)
    w_dn = _full_weight(hidden, inner, 12).double().requires_grad_(True)
    if dtype != torch.float32:
        with torch.no_grad():
            w_up.copy_(w_up.to(dtype).double())
            w_dn.copy_(w_dn.to(dtype).double())
    xr = x_full.to(dtype).double().requires_grad_(True)
    yr = torch.nn.functional.gelu(xr @ w_up.t()) @ w_dn.t()
    yr.backward(gy_full.to(dtype).double())
    sl = slice(rank * rows, (rank + 1) * rows)
    n_in = inner // world
    torch.testing.assert_close(y.detach().double().cpu(), yr[sl].detach(), rtol=tol, atol=tol)
    torch.testing.assert_close(x.grad.double().cpu(), xr.grad[sl], rtol=tol, atol=tol)
    torch.testing.assert_close(mlp.up.weight.grad.double().cpu(), w_up.grad[rank * n_in:(rank + 1) * n_in], rtol=tol, atol=tol * 4)
    torch.testing.assert_close(mlp.down.weight.grad.double().cpu(), w_dn.grad[:, rank * n_in:(rank + 1) * n_in], rtol=tol, atol=tol * 4)
    dist.barrier()


def test_parallel_mlp_cpu_world2():
    run_ranks(_tp_mlp, world=2, args=("cpu", 64, 32, 96, "float32", 1e-5))


def test_parallel_mlp_cpu_world4_bf16():
    run_ranks(_tp_mlp, world=4, args=("cpu", 64, 32, 96, "bfloat16", 6e-2))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_parallel_mlp_cuda_fused_forward():
    # 128 x world rows so that the fused all_gather + GEMM and GEMM + reduce_scatter kernels are taken
    w = min(torch.cuda.device_count(), 8)
    run_ranks(_tp_mlp, world=w, device="cuda", args=("cuda", 128 * w * 2, 256, 512, "bfloat16", 8e-2),
              env={"NCCL_NVLS_ENABLE": "0"}, timeout=150)
