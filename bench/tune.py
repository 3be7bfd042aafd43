"""Measures the algorithm crossovers of the CUDA collectives on the machine at hand and writes
the line of this world size into a tuning file for CCL_TUNE_FILE.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/tune.py --out ccl_tune.txt

* all_reduce: one-shot (every rank pushes its whole tensor to every peer) against two-shot
  (reduce-scatter then all-gather) and, when the arenas are bound to an NVLink multicast object
  (CCL_NVLS=1), the in-switch reduction, from 32 KB to 64 MB; `oneshot_max_bytes` is the largest
  size up to which one-shot is never slower than the best of the others, `nvls_min_bytes` the
  size from which the switch kernel is never slower than the peer-load kernels.
* all_reduce on symmetric tensors: the zero-copy kernels against the staged ones;
  `symm_min_bytes` is the size from which zero-copy is never slower.
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


def first_win(sizes, first, second):
    """Smallest size from which `first` is never slower than `second` (0: never)."""
    best = 0
    for s, a, b in reversed(list(zip(sizes, first, second))):
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

    import torch_ccl_b200

    cfg = be.cuda_comm_config(probe)
    have_nvls = bool(cfg["nvls_available"])
    sizes = [32 << 10 << i for i in range(12)]  # 32 KB .. 64 MB
    one, two, nvls, symm, staged = [], [], [], [], []
    sym_buf = torch_ccl_b200.symm_empty(sizes[-1] // 2, torch.bfloat16)
    for size in sizes:
        t = torch.ones(size // 2, device=dev, dtype=torch.bfloat16)
        be.set_cuda_tuning(probe, {"oneshot_max_bytes": BIG, "algo": 1, "symm_min_bytes": BIG})
        one.append(timed(lambda: be.fused_allreduce(t, 1.0), dev))
        be.set_cuda_tuning(probe, {"algo": 2})
        two.append(timed(lambda: be.fused_allreduce(t, 1.0), dev))
        row = {"op": "all_reduce", "bytes": size, "oneshot_us": round(one[-1], 2), "twoshot_us": round(two[-1], 2)}
        if have_nvls:
            be.set_cuda_tuning(probe, {"algo": 3})
            nvls.append(timed(lambda: be.fused_allreduce(t, 1.0), dev))
            row["nvls_us"] = round(nvls[-1], 2)
        st = sym_buf[: size // 2]
        st.fill_(1.0)
        best_algo = min([(one[-1], 1), (two[-1], 2)] + ([(nvls[-1], 3)] if have_nvls else []))[1]
        be.set_cuda_tuning(probe, {"algo": best_algo})  # staged, best algorithm, symmetric tensor
        staged.append(timed(lambda: be.fused_allreduce(st, 1.0), dev))
        be.set_cuda_tuning(probe, {"algo": 0, "symm_min_bytes": 0})  # zero-copy
        symm.append(timed(lambda: be.fused_allreduce(st, 1.0), dev))
        row["symm_zero_copy_us"] = round(symm[-1], 2)
        row["symm_staged_us"] = round(staged[-1], 2)
        rows.append(row)
        del t
    be.set_cuda_tuning(probe, {"algo": 0})
    others = [min(a, b) for a, b in zip(two, nvls)] if have_nvls else two
    oneshot_max = crossover(sizes, one, others)
    peer = [min(a, b) for a, b in zip(one, two)]
    nvls_min = first_win(sizes, nvls, peer) if have_nvls else 0
    symm_min = first_win(sizes, symm, staged)
    del sym_buf

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
        line = "%d oneshot_max_bytes=%d ag_push_max_bytes=%d" % (world, max(1, oneshot_max), max(1, ag_push_max))  # 0 would mean "built-in default"
        if nvls_min:
            line += " nvls_min_bytes=%d" % nvls_min
        if symm_min:
            line += " symm_min_bytes=%d" % symm_min
        keep.append(line)
        with open(a.out, "w") as f:
            f.write("\n".join(keep) + "\n")
        print(json.dumps({"world": world, "oneshot_max_bytes": oneshot_max, "ag_push_max_bytes": ag_push_max, "nvls_min_bytes": nvls_min,
                          "symm_min_bytes": symm_min, "nvls_available": have_nvls, "heap_multicast": bool(be.symm_heap_info(probe)["multicast"]),
                          "rows": rows}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
