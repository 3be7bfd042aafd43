"""CPU tensors: the shared-memory `ccl` backend against gloo on the same machine, all_reduce /
all_gather / reduce_scatter / all_to_all / broadcast from 1 KB to 64 MB, fp32.

    python bench/cpu_sweep.py --world 4 [--max-mb 64]

Wall-clock per call (barrier before, max over ranks), median of the timed iterations. gloo is
the only other CPU backend in the image; the reference's own CPU path is oneCCL, which cannot
be installed here.
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, group, iters):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier(group=group)
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    t = torch.tensor([statistics.median(ts)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t) * 1e6


def worker(rank, world, args):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(args.port))
    torch.set_num_threads(1)
    import oneccl_bindings_for_pytorch  # noqa: F401

    dist.init_process_group("ccl", rank=rank, world_size=world)
    groups = {"ccl": None, "gloo": dist.new_group(backend="gloo")}
    rows = []
    size = 1 << 10
    while size <= args.max_mb << 20:
        n = size // 4
        iters = 30 if size <= (1 << 20) else 8
        row = {"bytes": size}
        for name, g in groups.items():
            x = torch.ones(n)
            out_full = torch.empty(n * world)
            full = torch.ones(n * world)
            part = torch.empty(n)
            r = {}
            r["all_reduce"] = timed(lambda: dist.all_reduce(x, group=g), g, iters)
            r["broadcast"] = timed(lambda: dist.broadcast(x, 0, group=g), g, iters)
            r["all_gather"] = timed(lambda: dist.all_gather_into_tensor(out_full, x, group=g), g, iters)
            if name == "ccl" or hasattr(dist, "reduce_scatter_tensor"):
                try:
                    r["reduce_scatter"] = timed(lambda: dist.reduce_scatter_tensor(part, full, group=g), g, iters)
                except Exception:
                    r["reduce_scatter"] = None
            try:
                r["all_to_all"] = timed(lambda: dist.all_to_all_single(out_full, full, group=g), g, iters)
            except Exception:
                r["all_to_all"] = None
            row[name] = {k: (round(v, 1) if v is not None else None) for k, v in r.items()}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        size *= 8
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--max-mb", type=int, default=64)
    ap.add_argument("--port", type=int, default=29661)
    a = ap.parse_args()
    mp.spawn(worker, args=(a.world, a), nprocs=a.world)


if __name__ == "__main__":
    main()
