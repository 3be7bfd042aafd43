"""Expert-parallel MoE layer in the Mixtral shape (8 experts, top-2 softmax router, hidden 4096,
expert FFN 14336 SwiGLU, bf16 N(0, 0.02) weights, N(0, 1) activations, 4096 tokens per GPU, experts
spread evenly over the GPUs) — the fused dispatch / combine kernels against an
all_to_all_single-based layer on torch's NCCL backend.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/moe_layer.py [--tokens 4096]

Both arms use the same expert GEMMs (this repository's tcgen05 GEMM) so the difference is the
exchange: ccl = moe_dispatch + moe_combine (routing permutation fused into the NVLink transfer);
nccl = argsort/permute + all_to_all_single (split sizes via a host sync, as in common MoE code) +
un-permute + weighted sum. Device-timed, max over ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oneccl_bindings_for_pytorch  # noqa: E402,F401
import torch_ccl_b200._C as C  # noqa: E402
from torch_ccl_b200 import get_backend  # noqa: E402


def expert_ffn(x, w13, w2, inter):
    """SwiGLU FFN of one expert on rows x [R, H]."""
    if x.shape[0] == 0:
        return x
    gu = torch.empty(x.shape[0], 2 * inter, device=x.device, dtype=torch.bfloat16)
    C.gemm_bf16_tn(x, w13, gu, False, 0, 1, 0)
    act = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    out = torch.empty(x.shape[0], x.shape[1], device=x.device, dtype=torch.bfloat16)
    C.gemm_bf16_tn(act.contiguous(), w2, out, False, 0, 1, 0)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("ccl", rank=rank, world_size=world)
    nccl = dist.new_group(backend="nccl")
    be = get_backend(None, "cuda")
    T, H, I, E, K = a.tokens, a.hidden, a.inter, a.experts, 2
    epr = E // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    router = (torch.randn(E, H, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) * 0.02).to(torch.bfloat16)
    w13 = [(torch.randn(2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(epr)]
    w2 = [(torch.randn(H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(epr)]
    cap_rows = min(world * T * K, be.moe_capacity(x) * world)
    out_x = torch.empty(cap_rows, H, device=dev, dtype=torch.bfloat16)
    meta = torch.empty(cap_rows, 3, device=dev, dtype=torch.int32)
    count = torch.zeros(16, device=dev, dtype=torch.int32)
    out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)

    def route():
        logits = (x @ router.t()).float()
        w, idx = torch.topk(torch.softmax(logits, -1), K, dim=-1)
        return (w / w.sum(-1, keepdim=True)).contiguous(), idx.to(torch.int32).contiguous()

    def run_experts(rows, local_expert):
        y = torch.empty_like(rows)
        for e in range(epr):
            sel = (local_expert == e).nonzero(as_tuple=True)[0] if epr > 1 else None
            if epr == 1:
                y = expert_ffn(rows, w13[0], w2[0], I)
            else:
                y[sel] = expert_ffn(rows[sel].contiguous(), w13[e], w2[e], I)
        return y

    def layer_ccl():
        gate, idx = route()
        be.fused_moe_dispatch(x, idx, out_x, meta, count, epr)
        n = int(count[0])  # the expert GEMMs need the row count on the host
        y = run_experts(out_x[:n], meta[:n, 2])
        be.fused_moe_combine(y, meta, count, gate, out)
        return out

    def layer_nccl():
        gate, idx = route()
        flat = idx.view(-1).long()
        order = torch.argsort(flat, stable=True)
        send = x[order // K]
        per_expert = torch.bincount(flat, minlength=E)
        send_split = per_expert.view(world, epr).sum(1)
        recv_split = torch.empty_like(send_split)
        dist.all_to_all_single(recv_split, send_split, group=nccl)
        recv_e = torch.empty(world * epr, dtype=per_expert.dtype, device=dev)
        dist.all_to_all_single(recv_e, per_expert, group=nccl)
        ss, rs = send_split.tolist(), recv_split.tolist()
        recv = torch.empty(sum(rs), H, device=dev, dtype=torch.bfloat16)
        dist.all_to_all_single(recv, send, rs, ss, group=nccl)
        local_expert = torch.repeat_interleave(torch.arange(world * epr, device=dev) % epr, recv_e)
        y = run_experts(recv, local_expert)
        back = torch.empty_like(send)
        dist.all_to_all_single(back, y, ss, rs, group=nccl)
        un = torch.empty_like(back)
        un[order] = back
        o = (un.view(T, K, H).float() * gate[:, :, None]).sum(1).to(torch.bfloat16)
        return o

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    o1 = layer_ccl().clone()
    o2 = layer_nccl()
    err = (o1.float() - o2.float()).abs().max().item()
    ms_ccl, ms_nccl = timeit(layer_ccl), timeit(layer_nccl)

    def exch_ccl():
        be.fused_moe_dispatch(x, idx0, out_x, meta, count, epr)
        be.fused_moe_combine(out_x, meta, count, gate0, out)

    gate0, idx0 = route()
    us_exch = timeit(exch_ccl) * 1e3
    if rank == 0:
        print(json.dumps({"bench": "moe_layer", "world": world, "tokens_per_gpu": T, "hidden": H, "ffn": I, "experts": E, "topk": K,
                          "ccl_layer_ms": round(ms_ccl, 3), "nccl_layer_ms": round(ms_nccl, 3), "speedup": round(ms_nccl / ms_ccl, 3),
                          "ccl_dispatch_plus_combine_us": round(us_exch, 1), "max_abs_diff_vs_nccl_arm": round(err, 4)}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
