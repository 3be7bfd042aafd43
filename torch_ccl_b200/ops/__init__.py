"""Fused collective + compute ops. Each runs on the CURRENT CUDA stream of the tensor's device
(so it can be captured in a CUDA graph) through the process group's peer-memory communicator."""
import torch

from .. import _C


def _backend(group, tensor):
    from .. import get_backend

    return get_backend(group, "cuda")


def allreduce_residual_rmsnorm(x, residual, weight, eps=1e-5, group=None, out=None):
    """residual <- residual + all_reduce(x); returns rmsnorm(residual) * weight, in one kernel."""
    out = torch.empty_like(x) if out is None else out
    _backend(group, x).fused_allreduce_residual_rmsnorm(x, residual, weight, out, eps)
    return out


def all_reduce_scaled(tensor, scale=1.0, group=None):
    """In-place SUM all_reduce with the result multiplied by `scale` in the same pass."""
    _backend(group, tensor).fused_allreduce(tensor, scale)
    return tensor


def reduce_scatter_cast(inp, out, scale=1.0, group=None):
    """out = scale * sum_ranks(piece of inp); `out` may be fp32 while `inp` is bf16/f16."""
    _backend(group, inp).fused_reduce_scatter_cast(inp, out, scale)
    return out


def all_gather_copy_out(shard, outs, group=None):
    """All-gather `shard` with rank p's piece written directly into outs[p]."""
    _backend(group, shard).fused_all_gather_copy_out(shard, list(outs))
    return outs


def gemm_reduce_scatter(a, b, group=None, out=None):
    """Row-parallel linear fused with its reduce-scatter: returns this rank's rows [M/W, N] of
    sum_ranks(a_rank[M, K_local] @ b_rank[N, K_local].T); tiles cross NVLink from the GEMM epilogue."""
    be = _backend(group, a)
    world = torch.distributed.get_world_size(group)
    if out is None:
        out = torch.empty(a.shape[0] // world, b.shape[0], device=a.device, dtype=torch.bfloat16)
    be.fused_gemm_rs(a, b, out)
    return out


def all_gather_gemm(a_shard, b, group=None, out=None):
    """All-gather fused with a column-parallel linear: returns all_gather(a_shard)[M, K] @ b[N, K].T;
    tiles of a shard start as soon as that shard has arrived."""
    be = _backend(group, a_shard)
    world = torch.distributed.get_world_size(group)
    if out is None:
        out = torch.empty(a_shard.shape[0] * world, b.shape[0], device=a_shard.device, dtype=torch.bfloat16)
    be.fused_ag_gemm(a_shard, b, out)
    return out


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
