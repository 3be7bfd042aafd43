"""Fused collective + compute ops of the `ccl` backend.

Every op is registered with the dispatcher as `torch.ops.ccl.<name>` (schema + CUDA kernel + Meta
kernel for shape inference), so it can be traced with fake tensors, exported and used under
`torch.compile`; the functions below are thin Python faces that pass the process group by name.
Each op runs on the CURRENT CUDA stream of the tensor's device (so it can be captured in a CUDA
graph) through the process group's peer-memory communicator."""
import torch
import torch.distributed as dist

from .. import _C


def _name(group):
    group = group if group is not None else dist.group.WORLD
    return group.group_name


def _backend(group, tensor):
    from .. import get_backend

    return get_backend(group, "cuda")


def allreduce_residual_rmsnorm(x, residual, weight, eps=1e-5, group=None, out=None):
    """residual <- residual + all_reduce(x); returns rmsnorm(residual) * weight, in one kernel."""
    if out is None:
        return torch.ops.ccl.allreduce_residual_rmsnorm(x, residual, weight, eps, _name(group))
    _backend(group, x).fused_allreduce_residual_rmsnorm(x, residual, weight, out, eps)
    return out


def gemm_allreduce_residual_rmsnorm(w_packed, x, residual, weight, eps=1e-5, group=None, out=None):
    """Row-parallel linear + all_reduce + residual add + RMSNorm in ONE kernel (tensor-parallel decode):
    residual <- residual + sum over ranks of x[rows, K_local] @ w[hidden, K_local].T; returns
    rmsnorm(residual) * weight. `w_packed` is pack_weight(w). Rows are limited (see
    `gemm_allreduce_residual_rmsnorm_max_rows`); larger inputs run the GEMM and
    allreduce_residual_rmsnorm separately."""
    if out is None:
        return torch.ops.ccl.gemm_ar_norm(w_packed, x, residual, weight, eps, _name(group))
    _backend(group, x).fused_gemm_ar_norm(w_packed, x, residual, weight, out, eps)
    return out


def all_reduce_scaled(tensor, scale=1.0, group=None):
    """In-place SUM all_reduce with the result multiplied by `scale` in the same pass."""
    torch.ops.ccl.all_reduce_scaled(tensor, scale, _name(group))
    return tensor


def reduce_scatter_cast(inp, out, scale=1.0, group=None):
    """out = scale * sum_ranks(piece of inp); `out` may be fp32 while `inp` is bf16/f16."""
    _backend(group, inp).fused_reduce_scatter_cast(inp, out, scale)
    return out


def all_gather_copy_out(shard, outs, group=None):
    """All-gather `shard` with rank p's piece written directly into outs[p]."""
    torch.ops.ccl.all_gather_copy_out(shard, list(outs), _name(group))
    return outs


def gemm_reduce_scatter(a, b, group=None, out=None):
    """Row-parallel linear fused with its reduce-scatter: returns this rank's rows [M/W, N] of
    sum_ranks(a_rank[M, K_local] @ b_rank[N, K_local].T); tiles cross NVLink from the GEMM epilogue."""
    if out is None:
        return torch.ops.ccl.gemm_reduce_scatter(a, b, _name(group))
    _backend(group, a).fused_gemm_rs(a, b, out)
    return out


def all_gather_gemm(a_shard, b, group=None, out=None):
    """All-gather fused with a column-parallel linear: returns all_gather(a_shard)[M, K] @ b[N, K].T;
    tiles of a shard start as soon as that shard has arrived."""
    if out is None:
        return torch.ops.ccl.all_gather_gemm(a_shard, b, _name(group))
    _backend(group, a_shard).fused_ag_gemm(a_shard, b, out)
    return out


def moe_dispatch(x, expert_idx, experts_per_rank, max_rows, group=None):
    """Expert-parallel dispatch: sends every (token, k) row of x to the rank that owns its expert.
    Returns (rows [max_rows, hidden], meta [max_rows, 3] = {source rank, source slot, local expert},
    count int32 [16]: count[0] = rows received). The order of the received rows of one source is
    not deterministic from run to run (positions come from an atomic counter); `meta` says which is which."""
    return torch.ops.ccl.moe_dispatch(x, expert_idx, experts_per_rank, max_rows, _name(group))


def moe_combine(y, meta, count, gate, group=None):
    """Expert-parallel combine: returns out[t] = sum_k gate[t, k] * (row of y that came from slot (t, k))."""
    return torch.ops.ccl.moe_combine(y, meta, count, gate, _name(group))


def pack_weight(w):
    """Re-lays a [rows, K] weight for streaming by the swap-AB GEMM: rows padded to a multiple of
    128 and K to a multiple of 64, stored as [rows/128][K/64][128][64] so that every 128x64 tile is
    one contiguous 16 KB block (a TMA box then reads whole DRAM pages instead of 128 strided
    128-byte pieces). Returns a [*, 64] bf16 tensor for `gemm_bf16_tn(..., a_tiled_rows=rows)`."""
    rows, k = w.shape
    rp, kp = (rows + 127) // 128 * 128, (k + 63) // 64 * 64
    if rp != rows or kp != k:
        w = torch.nn.functional.pad(w, (0, kp - k, 0, rp - rows))
    return w.view(rp // 128, 128, kp // 64, 64).permute(0, 2, 1, 3).contiguous().view(-1, 64)


def unpack_weight(packed, rows, k):
    """Inverse of pack_weight."""
    rp, kp = (rows + 127) // 128 * 128, (k + 63) // 64 * 64
    w = packed.view(rp // 128, kp // 64, 128, 64).permute(0, 2, 1, 3).reshape(rp, kp)
    return w[:rows, :k]


def gemm_bf16_tn(a, b, out=None, trans_out=False, dual_off=0, splitk=0, bn=0, out_dtype=None, a_tiled_rows=0):
    """out = a @ b.T on tcgen05 tensor cores (bf16 operands, fp32 accumulation)."""
    m = a_tiled_rows if a_tiled_rows > 0 else (dual_off if dual_off > 0 else a.shape[0])
    n = b.shape[0]
    if out is None:
        shape = (n, m) if trans_out else (m, n)
        out = torch.empty(shape, device=a.device, dtype=out_dtype or torch.bfloat16)
    _C.gemm_bf16_tn(a, b, out, trans_out, dual_off, splitk, bn, a_tiled_rows)
    return out
