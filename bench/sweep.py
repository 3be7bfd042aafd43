"""Collective bus-bandwidth / latency sweep: the `ccl` backend against torch's NCCL backend on the
same GPUs (the counterpart of the reference's size-sweep script tests/ddp_allreduce.py:73-117,
which can also run the same sweep on `nccl`).

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/sweep.py \
        [--ops all_reduce,reduce_scatter,all_gather,all_to_all] [--dtypes bf16,fp32] \
        [--min-bytes 8192] [--max-bytes 1073741824] [--iters 20] [--out sweep.json]

Sizes are bytes of the full per-rank tensor S (the large side of the op). Timing: CUDA events
around `iters` back-to-back calls after warm-up, max over ranks. Between sizes the buffers cycle
through a pool larger than L2 for messages below 128 MB. Reported: time per call, algBW = S/t and
busBW = algBW * 2(N-1)/N (all_reduce) or algBW * (N-1)/N (the others).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oneccl_bindings_for_pytorch  # noqa: E402,F401

DT = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}


def make_op(name, group, n_elems, dtype, world, dev, symmetric=False):
    """Returns (callable taking a buffer index, number of pooled buffers). `symmetric`: the buffers a
    peer touches (all_reduce tensor, reduce_scatter input, all_gather output) come from the group's
    symmetric heap, so the `ccl` backend runs its zero-copy kernels."""
    pool = max(1, min(8, int(256e6 // max(1, n_elems * dtype.itemsize)) + 1))
    g = torch.Generator(device=dev).manual_seed(7)

    def rand(n, symm):
        t = torch.randn(n, device=dev, generator=g).to(dtype)
        if symm:
            import torch_ccl_b200

            st = torch_ccl_b200.symm_empty(n, dtype, group=group)
            st.copy_(t)
            return st
        return t

    if name == "all_reduce":
        bufs = [rand(n_elems, symmetric) for _ in range(pool)]
        return (lambda i: dist.all_reduce(bufs[i % pool], group=group)), pool
    if name == "reduce_scatter":
        n = n_elems // world * world
        ins = [rand(n, symmetric) for _ in range(pool)]
        out = torch.empty(n // world, device=dev, dtype=dtype)
        return (lambda i: dist.reduce_scatter_tensor(out, ins[i % pool], group=group)), pool
    if name == "all_gather":
        n = n_elems // world * world
        ins = [rand(n // world, False) for _ in range(pool)]
        out = rand(n, symmetric)
        return (lambda i: dist.all_gather_into_tensor(out, ins[i % pool], group=group)), pool
    if name == "all_to_all":
        n = n_elems // world * world
        ins = [torch.randn(n, device=dev, generator=g).to(dtype) for _ in range(pool)]
        out = torch.empty(n, device=dev, dtype=dtype)
        return (lambda i: dist.all_to_all_single(out, ins[i % pool], group=group)), pool
    raise ValueError(name)


def time_op(fn, iters, warmup, group, dev):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize(dev)
    dist.barrier(group=group)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item()) * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="all_reduce,reduce_scatter,all_gather,all_to_all")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--min-bytes", type=int, default=8 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--step", type=int, default=2, help="size multiplier between points")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--backends", default="ccl,nccl")
    ap.add_argument("--out", default="")
    ap.add_argument("--symmetric", action="store_true",
                    help="add a third arm: ccl on tensors from the symmetric heap (zero-copy kernels; set CCL_SYMM_HEAP_MB large enough)")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("ccl", rank=rank, world_size=world)
    groups = {}
    for b in args.backends.split(","):
        groups[b] = dist.group.WORLD if b == "ccl" else dist.new_group(backend=b)

    rows = []
    for op in args.ops.split(","):
        for dn in args.dtypes.split(","):
            dtype = DT[dn]
            size = args.min_bytes
            while size <= args.max_bytes:
                n = size // dtype.itemsize
                row = {"op": op, "dtype": dn, "bytes": size, "world": world}
                for b, grp in groups.items():
                    fn, _ = make_op(op, grp, n, dtype, world, dev)
                    iters = max(3, min(args.iters, int(2e9 // size) + 3))
                    t = time_op(fn, iters, args.warmup, grp, dev)
                    alg = size / t / 1e9
                    bus = alg * (2 * (world - 1) / world if op == "all_reduce" else (world - 1) / world)
                    row[b] = {"us": round(t * 1e6, 2), "algbw_GBps": round(alg, 2), "busbw_GBps": round(bus, 2)}
                    del fn
                    torch.cuda.empty_cache()
                if args.symmetric and op != "all_to_all" and "ccl" in groups:
                    fn, _ = make_op(op, groups["ccl"], n, dtype, world, dev, symmetric=True)
                    iters = max(3, min(args.iters, int(2e9 // size) + 3))
                    t = time_op(fn, iters, args.warmup, groups["ccl"], dev)
                    alg = size / t / 1e9
                    bus = alg * (2 * (world - 1) / world if op == "all_reduce" else (world - 1) / world)
                    row["ccl_symmetric"] = {"us": round(t * 1e6, 2), "algbw_GBps": round(alg, 2), "busbw_GBps": round(bus, 2)}
                    del fn
                    torch.cuda.empty_cache()
                if "ccl" in row and "nccl" in row:
                    row["speedup_vs_nccl"] = round(row["nccl"]["us"] / row["ccl"]["us"], 3)
                if "ccl_symmetric" in row and "nccl" in row:
                    row["symmetric_speedup_vs_nccl"] = round(row["nccl"]["us"] / row["ccl_symmetric"]["us"], 3)
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
                size *= args.step
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"world": world, "rows": rows}, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
