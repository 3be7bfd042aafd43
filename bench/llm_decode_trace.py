"""The two decode-shaped all_reduce workloads the reference ships without results, with an NCCL
arm and value checks:

  trace        140 all_reduces of 458 752 fp16 elements (prompt phase) followed by 31 x 140 of
               14 336 elements (token phase), 10 repeats, device-timed per repeat
               (src/gpu/allreduce.cpp:70-97 of intel/torch-ccl, its stand-alone MPI benchmark)
  interleaved  N rounds of { elementwise work on a large tensor ; all_reduce of 14 336 fp16
               elements ; average ; read one value back to the host }, wall-clocked because the
               host read is part of the loop (tests/test_allreduce.py:49-76: 2240 rounds on a
               72 Mi-element tensor, then an element-wise comparison with a CPU recomputation)

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/llm_decode_trace.py [--mode trace|interleaved]
    python bench/llm_decode_trace.py --device cpu --small        # 2 CPU ranks, reduced counts (script self-check)
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def sync(dev):
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)


def run_trace(group, dev, dtype, small):
    world = dist.get_world_size(group)
    big_n, small_n = (4096, 256) if small else (14336 * 32, 14336)
    n_big, n_small, repeats = (4, 8, 2) if small else (140, 31 * 140, 10)
    big = torch.ones(big_n, device=dev, dtype=dtype)
    tok = torch.ones(small_n, device=dev, dtype=dtype)

    def one_pass():
        for _ in range(n_big):
            big.fill_(1.0)
            dist.all_reduce(big, group=group)
        for _ in range(n_small):
            tok.fill_(1.0)
            dist.all_reduce(tok, group=group)

    one_pass()
    sync(dev)
    assert float(big[0]) == world and float(tok[-1]) == world
    times = []
    for _ in range(repeats):
        dist.barrier(group=group)
        sync(dev)
        if dev.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            one_pass()
            e1.record()
            sync(dev)
            ms = e0.elapsed_time(e1)
        else:
            t0 = time.perf_counter()
            one_pass()
            ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        times.append(float(t))
    return {"all_reduces_per_pass": n_big + n_small, "ms_per_pass_mean": round(sum(times) / len(times), 3), "ms_per_pass_min": round(min(times), 3)}


def run_interleaved(group, dev, dtype, small):
    world = dist.get_world_size(group)
    count = 256 if small else 14336
    rounds = 20 if small else 2240
    big_rows = 8 if small else 2048  # x count elements of elementwise work per round
    a = torch.zeros(big_rows, count, device=dev, dtype=torch.float32)
    data = torch.full((count,), 0.1, device=dev, dtype=dtype)
    for _ in range(3):  # untimed: communicator bring-up, allocator warm-up
        dist.all_reduce(data, group=group)
        data /= world
    data.fill_(0.1)
    dist.barrier(group=group)
    sync(dev)
    t0 = time.perf_counter()
    for _ in range(rounds):
        a[0] += data.float() * 0.1
        a += 0.01
        dist.all_reduce(data, group=group)
        data /= world
        _ = data[:1].cpu()  # the reference reads the tensor back every round
    sync(dev)
    span = time.perf_counter() - t0
    # every rank holds the same data, so the average returns the input: recompute on the CPU
    ref = torch.zeros(1, dtype=torch.float32)
    d = torch.full((1,), 0.1, dtype=dtype)
    for _ in range(rounds):
        ref += d.float() * 0.1
        ref += 0.01
        d = (d * world) / world if dtype == torch.float32 else ((d.float() * world).to(dtype).float() / world).to(dtype)
    ok = torch.allclose(a[0].cpu(), ref.expand(count), rtol=1e-3, atol=1e-3)
    t = torch.tensor([span], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return {"rounds": rounds, "seconds": round(float(t), 4), "us_per_round": round(float(t) / rounds * 1e6, 1), "matches_cpu": bool(ok)}


def worker(rank, world, args, spawned):
    if spawned:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT="29641")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    import oneccl_bindings_for_pytorch  # noqa: F401

    if args.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dev = torch.device("cpu")
    dist.init_process_group("ccl", rank=rank, world_size=world)
    dtype = torch.float16 if args.device == "cuda" else torch.float32
    fn = run_trace if args.mode == "trace" else run_interleaved
    out = {"bench": "llm_decode_trace", "mode": args.mode, "world": world, "device": args.device, "dtype": str(dtype).split(".")[-1]}
    out["ccl"] = fn(None, dev, dtype, args.small)
    if args.device == "cuda" and not args.no_nccl:
        nccl = dist.new_group(backend="nccl")
        out["nccl"] = fn(nccl, dev, dtype, args.small)
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="trace", choices=["trace", "interleaved"])
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--small", action="store_true", help="reduced counts (self-check of the script)")
    ap.add_argument("--no-nccl", action="store_true")
    args = ap.parse_args()
    if "RANK" in os.environ:
        worker(0, 0, args, False)
    else:
        world = 2 if args.device == "cpu" else torch.cuda.device_count()
        mp.spawn(worker, args=(world, args, True), nprocs=world)


if __name__ == "__main__":
    main()
