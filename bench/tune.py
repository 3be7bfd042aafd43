"""Measures the algorithm crossovers of the CUDA collectives on the machine at hand and writes
the line of this world size into a tuning file for CCL_TUNE_FILE.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/tune.py --out ccl_tune.txt

* all_reduce: one-shot (every rank pushes its whole tensor to every peer) against two-shot
  (reduce-scatter then all-gather) from 32 KB to 16 MB; `oneshot_max_bytes` is the largest size
  up to which one-shot is never slower.
* all_gather: push against pull per piece size; `ag_push_max_bytes` likewise.

Timings are device-side (CUDA graph of 20 calls between two events), max over ranks, so every
rank derives the same numbers. Lines of other world sizes already in the file are kept.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oneccl_bindings_for_pytorch  # noqa: E402,F401
from torch_ccl_b200 import get_backend  # noqa: E402

BIG = 1 << 40


def timed(fn, dev, iters=20):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for _ in range(iters):
            fn()
    dist.barrier()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / iters * 1e3
        best = us if best is None else min(best, us)
    t = torch.tensor([best], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def crossover(sizes, first, second):
    """Largest size up to which `first` was never slower than `second` (0 if it never wins)."""
    best = 0
    for s, a, b in zip(sizes, first, second):
        if a <= b * 1.02:
            best = s
        else:
            break
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="ccl_tune.txt")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("ccl", rank=rank, world_size=world)
    be = get_backend(None, "cuda")
    probe = torch.ones(8, device=dev)
    dist.all_reduce(probe)
    rows = []

    sizes = [32 << 10 << i for i in range(10)]  # 32 KB .. 16 MB
    one, two = [], []
    for size in sizes:
        t = torch.ones(size // 2, device=dev, dtype=torch.bfloat16)
        be.set_cuda_tuning(probe, {"oneshot_max_bytes": BIG})
        one.append(timed(lambda: be.fused_allreduce(t, 1.0), dev))
        be.set_cuda_tuning(probe, {"oneshot_max_bytes": 1})
        two.append(timed(lambda: be.fused_allreduce(t, 1.0), dev))
        rows.append({"op": "all_reduce", "bytes": size, "oneshot_us": round(one[-1], 2), "twoshot_us": round(two[-1], 2)})
    oneshot_max = crossover(sizes, one, two)

    pieces = [8 << 10 << i for i in range(9)]  # 8 KB .. 2 MB per rank
    push, pull = [], []
    for piece in pieces:
        src = torch.ones(piece // 2, device=dev, dtype=torch.bfloat16)
        outs = list(torch.empty(world * piece // 2, device=dev, dtype=torch.bfloat16).chunk(world))
        be.set_cuda_tuning(probe, {"ag_push_max_bytes": BIG})
        push.append(timed(lambda: be.fused_all_gather_copy_out(src, outs), dev))
        be.set_cuda_tuning(probe, {"ag_push_max_bytes": 0})
        pull.append(timed(lambda: be.fused_all_gather_copy_out(src, outs), dev))
        rows.append({"op": "all_gather", "piece_bytes": piece, "push_us": round(push[-1], 2), "pull_us": round(pull[-1], 2)})
    ag_push_max = crossover(pieces, push, pull)

    if rank == 0:
        keep = []
        if os.path.exists(a.out):
            for line in open(a.out):
                head = line.split("#")[0].split()
                if not head or head[0] != str(world):
                    keep.append(line.rstrip("\n"))
        keep.append("%d oneshot_max_bytes=%d ag_push_max_bytes=%d" % (world, max(1, oneshot_max), max(1, ag_push_max)))  # 0 would mean "built-in default"
        with open(a.out, "w") as f:
            f.write("\n".join(keep) + "\n")
        print(json.dumps({"world": world, "oneshot_max_bytes": oneshot_max, "ag_push_max_bytes": ag_push_max, "rows": rows}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
