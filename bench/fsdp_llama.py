"""Full-shard (ZeRO-3) training step of a Llama-architecture model: bf16 parameters and compute,
fp32 gradient reduction and master weights, sequence 2048, micro-batch 1 per GPU, uniform random
token ids. Arms (`--arms`, comma separated):

  ccl          the fused-collective engine of this repository (`torch_ccl_b200.parallel.fsdp`: all_gather with
               direct copy-out, reduce_scatter with fused average + fp32 cast) on the `ccl` backend
  nccl         the same engine and schedule on plain torch.distributed calls over torch's NCCL backend
  fsdp2        stock `torch.distributed.fsdp.fully_shard` (bf16 parameters, fp32 reduce, activation
               checkpointing per layer) over NCCL - what a user of the stock stack runs
  fsdp2_ccl    the same stock fully_shard model over the `ccl` backend (the usage the reference tests:
               tests/test_fsdp.py:153 of intel/torch-ccl)

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/fsdp_llama.py \
        [--layers 32] [--hidden 4096] [--ffn 11008] [--seq 2048] [--steps 5] [--comm-blocks 48]

Device-timed (CUDA events), max over ranks; prints step time and tokens/s of the whole job.
"""
import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oneccl_bindings_for_pytorch  # noqa: E402,F401
from torch_ccl_b200.parallel.fsdp import FullyShardedSequential  # noqa: E402


class RMSNorm(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class Block(nn.Module):
    def __init__(self, d, heads, ffn):
        super().__init__()
        self.heads = heads
        self.n1, self.n2 = RMSNorm(d), RMSNorm(d)
        self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.o = nn.Linear(d, d, bias=False)
        self.gu = nn.Linear(d, 2 * ffn, bias=False)
        self.down = nn.Linear(ffn, d, bias=False)

    def forward(self, x):
        B, S, D = x.shape
        hd = D // self.heads
        q, k, v = self.qkv(self.n1(x)).view(B, S, 3, self.heads, hd).unbind(2)
        pos = torch.arange(S, device=x.device, dtype=torch.float32)
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd))
        ang = pos[:, None] * inv[None]
        cos, sin = ang.cos()[None, :, None, :].to(x.dtype), ang.sin()[None, :, None, :].to(x.dtype)

        def rope(t):
            t1, t2 = t[..., : hd // 2], t[..., hd // 2:]
            return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1)

        a = F.scaled_dot_product_attention(rope(q).transpose(1, 2), rope(k).transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(B, S, D))
        g, u = self.gu(self.n2(x)).chunk(2, -1)
        return x + self.down(F.silu(g) * u)


class Embed(nn.Module):
    def __init__(self, vocab, d):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)

    def forward(self, ids):
        return self.emb(ids)


class Head(nn.Module):
    def __init__(self, vocab, d):
        super().__init__()
        self.norm = RMSNorm(d)
        self.out = nn.Linear(d, vocab, bias=False)

    def forward(self, x):
        return self.out(self.norm(x))


def build(args, dev):
    torch.manual_seed(0)
    mods = [Embed(args.vocab, args.hidden)] + [Block(args.hidden, args.heads, args.ffn) for _ in range(args.layers)] + [Head(args.vocab, args.hidden)]
    for m in mods:
        m.to(dev)
        for p in m.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02)
    return mods


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--arms", default="ccl,nccl")
    ap.add_argument("--symmetric", action="store_true", help="ccl arm: parameter / gradient buffers from the symmetric heap (zero-copy collectives)")
    ap.add_argument("--comm-blocks", type=int, default=0, help="CTA cap of the ccl collectives while they overlap compute (0: library default)")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("ccl", rank=rank, world_size=world)
    results = {}
    nccl_group = None
    for arm in a.arms.split(","):
        if arm in ("nccl", "fsdp2") and nccl_group is None:
            nccl_group = dist.new_group(backend="nccl")
        g = torch.Generator().manual_seed(1 + rank)
        mods = build(a, dev)
        if arm in ("ccl", "nccl"):
            engine = FullyShardedSequential(mods, group=None if arm == "ccl" else nccl_group, comm="ccl" if arm == "ccl" else "c10d",
                                            comm_blocks=(a.comm_blocks or None) if arm == "ccl" else None,
                                            symmetric=a.symmetric and arm == "ccl")
            opt = torch.optim.AdamW(engine.master_params(), lr=1e-4, fused=True)

            def step():
                ids = torch.randint(0, a.vocab, (1, a.seq), generator=g).to(dev)
                labels = torch.randint(0, a.vocab, (1, a.seq), generator=g).to(dev)
                logits = engine(ids)
                loss = F.cross_entropy(logits.float().view(-1, a.vocab), labels.view(-1))
                loss.backward()
                engine.master_params()
                opt.step()
                engine.after_step()
                return loss
        else:
            from torch.distributed.device_mesh import DeviceMesh
            from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
            from torch.utils.checkpoint import checkpoint

            grp = nccl_group if arm == "fsdp2" else dist.group.WORLD
            mesh = DeviceMesh.from_group(grp, "cuda", mesh=list(range(world)))
            mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
            for m in mods:
                fully_shard(m, mesh=mesh, mp_policy=mp)
            engine = nn.ModuleList(mods)
            opt = torch.optim.AdamW(engine.parameters(), lr=1e-4, fused=True)

            def run_model(ids):
                x = mods[0](ids)
                for blk in mods[1:-1]:
                    x = checkpoint(blk, x, use_reentrant=False)  # recompute activations per layer, like the engine above
                return mods[-1](x)

            def step():
                ids = torch.randint(0, a.vocab, (1, a.seq), generator=g).to(dev)
                labels = torch.randint(0, a.vocab, (1, a.seq), generator=g).to(dev)
                logits = run_model(ids)
                loss = F.cross_entropy(logits.float().view(-1, a.vocab), labels.view(-1))
                loss.backward()
                opt.step()
                opt.zero_grad(set_to_none=True)
                return loss

        for _ in range(a.warmup):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            loss = step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[arm] = {"ms_per_step": round(float(t), 2), "tokens_per_s": round(world * a.seq / (float(t) * 1e-3), 1),
                        "final_loss": round(float(loss), 4)}
        del engine, opt, mods, step
        torch.cuda.empty_cache()
    if rank == 0:
        out = {"bench": "fsdp_llama", "world": world, "layers": a.layers, "hidden": a.hidden, "ffn": a.ffn, "seq": a.seq,
               "micro_batch": 1, "dtype": "bf16 params/compute, fp32 reduce + master"}
        out.update(results)
        out["comm_blocks"] = a.comm_blocks
        out["symmetric"] = a.symmetric
        if "ccl" in results and "nccl" in results:
            out["speedup_vs_nccl"] = round(results["nccl"]["ms_per_step"] / results["ccl"]["ms_per_step"], 3)
        if "ccl" in results and "fsdp2" in results:
            out["speedup_vs_torch_fsdp2_nccl"] = round(results["fsdp2"]["ms_per_step"] / results["ccl"]["ms_per_step"], 3)
        print(json.dumps(out))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
