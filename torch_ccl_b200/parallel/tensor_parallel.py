"""Megatron-style tensor-parallel linear layers with sequence parallelism, on any process group.

Between layers the activations are sharded over the sequence: `[S/W, hidden]` per rank. A
transformer block is then

    ColumnParallelLinear   all_gather(x over S) -> x @ W_col_r^T       (output `[S, out/W]`)
    RowParallelLinear      y_r @ W_row_r^T -> reduce_scatter over S     (output `[S/W, out]`)

and the backward pass mirrors it (the gradient of an all_gather is a reduce_scatter and vice
versa). The forward of both layers maps onto the fused ops of this package on CUDA - all_gather
overlapped with the GEMM (`ops.all_gather_gemm`) and GEMM overlapped with the reduce_scatter
(`ops.gemm_reduce_scatter`) - when the shapes fit their tiling (bf16, rows a multiple of
128 x world); otherwise, and always on CPU tensors, plain torch.distributed collectives are used,
which is also what the tests compare against a dense single-process layer.

The reference ships no model or layer code; it only provides the collectives such layers call
(`_allgather_base`, `_reduce_scatter_base`: src/ProcessGroupCCL.cpp, src/gpu/dpcpp_ccl.cpp:971-1019,
1147-1192 of intel/torch-ccl).
"""
import math

import torch
import torch.distributed as dist
import torch.nn as nn


def _world(group):
    return dist.get_world_size(group)


def _all_gather_rows(x, group):
    out = torch.empty((x.shape[0] * _world(group),) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x, group):
    w = _world(group)
    out = torch.empty((x.shape[0] // w,) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    return out


def _fused_ok(x, weight, group, rows_total):
    """The fused GEMM + collective kernels take bf16 CUDA operands, 128 x world row blocks and
    16-byte aligned K; only the `ccl` backend has them."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16):
        return False
    if dist.get_backend(group) != "ccl":
        return False
    w = _world(group)
    if not (rows_total % (128 * w) == 0 and weight.shape[1] % 8 == 0 and weight.shape[0] % 16 == 0 and x.dim() == 2):
        return False
    # the kernels stage one full operand / result in one half of the communicator's arena (CCL_ARENA_MB sets its size)
    from .. import get_backend

    staged = rows_total * max(weight.shape[0], weight.shape[1]) * 2
    return staged <= get_backend(group, "cuda").fused_gemm_capacity_bytes(x)


class _GatherMatmul(torch.autograd.Function):
    """y = all_gather_rows(x) @ w^T.  dx = reduce_scatter_rows(dy @ w), dw = dy^T @ all_gather_rows(x)."""

    @staticmethod
    def forward(ctx, x, w, group, fused):
        ctx.group = group
        ctx.save_for_backward(x, w)
        if fused and _fused_ok(x, w, group, x.shape[0] * _world(group)):
            from .. import ops

            return ops.all_gather_gemm(x.contiguous(), w.contiguous(), group=group)
        return _all_gather_rows(x, group) @ w.t()

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = _reduce_scatter_rows(dy @ w, ctx.group) if ctx.needs_input_grad[0] else None
        dw = dy.t() @ _all_gather_rows(x, ctx.group) if ctx.needs_input_grad[1] else None  # x is re-gathered, not kept
        return dx, dw, None, None


class _MatmulScatter(torch.autograd.Function):
    """y = reduce_scatter_rows(x @ w^T).  dx = all_gather_rows(dy) @ w, dw = all_gather_rows(dy)^T @ x."""

    @staticmethod
    def forward(ctx, x, w, group, fused):
        ctx.group = group
        ctx.save_for_backward(x, w)
        if fused and _fused_ok(x, w, group, x.shape[0]):
            from .. import ops

            return ops.gemm_reduce_scatter(x.contiguous(), w.contiguous(), group=group)
        return _reduce_scatter_rows(x @ w.t(), group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dyf = _all_gather_rows(dy, ctx.group)
        dx = dyf @ w if ctx.needs_input_grad[0] else None
        dw = dyf.t() @ x if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def _init_shard(out_features, in_features, dim, rank, world, seed, device, dtype):
    """The rank's shard of one deterministic full weight (the same on every rank for a seed)."""
    g = torch.Generator().manual_seed(seed)
    full = torch.empty(out_features, in_features).uniform_(-1.0, 1.0, generator=g) / math.sqrt(in_features)
    n = full.shape[dim] // world
    shard = full.narrow(dim, rank * n, n)
    return shard.to(device=device, dtype=dtype).contiguous()


class ColumnParallelLinear(nn.Module):
    """`[S/W, in] -> [S, out/W]`: gathers the sequence shards and applies this rank's output columns."""

    def __init__(self, in_features, out_features, group=None, seed=0, device=None, dtype=torch.float32, fused=True):
        super().__init__()
        w, r = _world(group), dist.get_rank(group)
        assert out_features % w == 0
        self.group, self.fused = group, fused
        self.weight = nn.Parameter(_init_shard(out_features, in_features, 0, r, w, seed, device, dtype))

    def forward(self, x):
        return _GatherMatmul.apply(x, self.weight, self.group, self.fused)


class RowParallelLinear(nn.Module):
    """`[S, in/W] -> [S/W, out]`: multiplies by this rank's input columns and reduce-scatters over the sequence."""

    def __init__(self, in_features, out_features, group=None, seed=1, device=None, dtype=torch.float32, fused=True):
        super().__init__()
        w, r = _world(group), dist.get_rank(group)
        assert in_features % w == 0
        self.group, self.fused = group, fused
        self.weight = nn.Parameter(_init_shard(out_features, in_features, 1, r, w, seed, device, dtype))

    def forward(self, x):
        return _MatmulScatter.apply(x, self.weight, self.group, self.fused)


class ParallelMLP(nn.Module):
    """Column-parallel up projection, GELU, row-parallel down projection: `[S/W, h] -> [S/W, h]` with one
    all_gather and one reduce_scatter per direction."""

    def __init__(self, hidden, inner, group=None, seed=0, device=None, dtype=torch.float32, fused=True):
        super().__init__()
        self.up = ColumnParallelLinear(hidden, inner, group, seed, device, dtype, fused)
        self.down = RowParallelLinear(inner, hidden, group, seed + 1, device, dtype, fused)

    def forward(self, x):
        return self.down(torch.nn.functional.gelu(self.up(x)))
