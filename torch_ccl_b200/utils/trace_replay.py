"""Replay of a recorded collective trace with value checks.

A trace is a CSV text with one collective per line: `op,numel,root` where op is one of
`allreduce`, `broadcast`, `reduce`, `allgather`, `reduce_scatter`, `alltoall`, `barrier` and root is
-1 for unrooted ops. This is the format of the ZeRO training trace that the reference replays as a
stress test (tests/DeepSpeed_test/DeepSpeed.csv with testccl_cpu.py:56-100 and testccl_gpu.py of
intel/torch-ccl: 491 ops, repeated 100 times, synchronous calls, no value checks — a hang and
crash detector). Here every op is also checked: the inputs are small integers that depend only on
(rank, op index, element index), so each rank can compute the expected result of every collective
locally and exactly, in any floating-point dtype, without a second communication library.

Run under torchrun (`python -m torch_ccl_b200.utils.trace_replay --trace t.csv --device cuda`) or
call `replay()` from a process group that is already initialised.
"""
import argparse
import io
import os
import time

import torch
import torch.distributed as dist

OPS = ("allreduce", "broadcast", "reduce", "allgather", "reduce_scatter", "alltoall", "barrier")


def parse_trace(text, world, scale=1, max_numel=None):
    """-> list of (op, numel, root). Sizes are divided by `scale` (at least 1 element) and capped."""
    out = []
    for ln, line in enumerate(io.StringIO(text), 1):
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        parts = [p.strip() for p in line.split(",")]
        if len(parts) != 3:
            raise ValueError("trace line %d: expected op,numel,root: %r" % (ln, line))
        op, numel, root = parts[0], int(parts[1]), int(parts[2])
        if op not in OPS:
            raise ValueError("trace line %d: unknown op %r" % (ln, op))
        if root >= world:
            raise ValueError("trace line %d: root %d outside a world of %d" % (ln, root, world))
        numel = max(1, numel // max(1, scale))
        if max_numel is not None:
            numel = min(numel, max_numel)
        out.append((op, numel, root))
    return out


def synthetic_zero_trace(world, layers=4, hidden=256, steps=2):
    """A ZeRO-1/2 shaped trace: parameter broadcast from rank 0 at start-up, then per step a
    gradient `reduce` to the rank that owns each bucket, an overflow / norm all_reduce of one
    element, and an all_gather of the updated partitions."""
    lines = ["allreduce,1,-1"]
    shapes = []
    for _ in range(layers):
        shapes += [3 * hidden * hidden, 3 * hidden, hidden * hidden, hidden, 4 * hidden * hidden, 4 * hidden,
                   4 * hidden * hidden, hidden, hidden, hidden]
    for n in shapes:
        lines.append("broadcast,%d,0" % n)
    for _ in range(steps):
        for i, n in enumerate(reversed(shapes)):
            lines.append("reduce,%d,%d" % (n, i % world))
        lines.append("allreduce,1,-1")
        lines.append("allreduce,%d,-1" % world)
        part = (sum(shapes) + world - 1) // world
        lines.append("allgather,%d,-1" % part)
        lines.append("barrier,1,-1")
    return "\n".join(lines) + "\n"


def _pattern(numel, rank, index, dtype, device):
    """Small integers that are exact in fp16 / bf16 even after a sum over 8 ranks."""
    base = torch.arange(numel, device=device, dtype=torch.int32).remainder_(5)
    return (base + (rank + 1) + (index % 3)).to(dtype)


def _sum_pattern(numel, world, index, dtype, device):
    base = torch.arange(numel, device=device, dtype=torch.int32).remainder_(5)
    return (base * world + world * (world + 1) // 2 + world * (index % 3)).to(dtype)


def replay(trace, rounds=1, device="cpu", dtype=torch.float16, group=None, check=True, async_op=False):
    """Runs `trace` (list from parse_trace) `rounds` times; returns {"ops", "seconds", "checked"}.

    Raises AssertionError naming the op index on the first wrong value."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    dev = torch.device(device)
    checked = 0
    t0 = time.perf_counter()
    for _ in range(rounds):
        for i, (op, n, root) in enumerate(trace):
            x = _pattern(n, rank, i, dtype, dev)
            expect = None
            if op == "allreduce":
                w = dist.all_reduce(x, group=group, async_op=async_op)
                got, expect = x, _sum_pattern(n, world, i, dtype, dev)
            elif op == "broadcast":
                w = dist.broadcast(x, dist.get_global_rank(group, root) if group is not None else root, group=group,
                                   async_op=async_op)
                got, expect = x, _pattern(n, root, i, dtype, dev)
            elif op == "reduce":
                w = dist.reduce(x, dist.get_global_rank(group, root) if group is not None else root, group=group,
                                async_op=async_op)
                got = x
                expect = _sum_pattern(n, world, i, dtype, dev) if rank == root else None
            elif op == "allgather":
                outs = [torch.empty_like(x) for _ in range(world)]
                w = dist.all_gather(outs, x, group=group, async_op=async_op)
                got = outs
                expect = [_pattern(n, r, i, dtype, dev) for r in range(world)]
            elif op == "reduce_scatter":
                full = _pattern(n * world, rank, i, dtype, dev)
                out = torch.empty(n, device=dev, dtype=dtype)
                w = dist.reduce_scatter_tensor(out, full, group=group, async_op=async_op)
                got = out
                expect = _sum_pattern(n * world, world, i, dtype, dev)[rank * n:(rank + 1) * n]
            elif op == "alltoall":
                full = _pattern(n * world, rank, i, dtype, dev)
                out = torch.empty_like(full)
                w = dist.all_to_all_single(out, full, group=group, async_op=async_op)
                got = out
                expect = torch.cat([_pattern(n * world, r, i, dtype, dev)[rank * n:(rank + 1) * n]
                                    for r in range(world)])
            else:
                w = dist.barrier(group=group, async_op=async_op)
                got = None
            if async_op and w is not None:
                w.wait()
            if check and expect is not None:
                if isinstance(expect, list):
                    ok = all(torch.equal(g, e) for g, e in zip(got, expect))
                else:
                    ok = torch.equal(got, expect)
                assert ok, "trace op %d (%s, %d elements, root %d): wrong result on rank %d" % (i, op, n, root, rank)
                checked += 1
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    return {"ops": rounds * len(trace), "seconds": time.perf_counter() - t0, "checked": checked}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--trace", help="CSV file (op,numel,root); default: a synthetic ZeRO trace")
    ap.add_argument("--rounds", type=int, default=10)
    ap.add_argument("--scale", type=int, default=1, help="divide every size by this")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--dtype", default="float16", choices=["float16", "bfloat16", "float32"])
    ap.add_argument("--backend", default="ccl")
    ap.add_argument("--no-check", action="store_true")
    args = ap.parse_args(argv)
    if args.backend == "ccl":
        import oneccl_bindings_for_pytorch  # noqa: F401
    if args.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(args.backend)
    world = dist.get_world_size()
    text = open(args.trace).read() if args.trace else synthetic_zero_trace(world)
    trace = parse_trace(text, world, scale=args.scale)
    res = replay(trace, rounds=args.rounds, device=args.device, dtype=getattr(torch, args.dtype), check=not args.no_check)
    if dist.get_rank() == 0:
        print("replayed %d ops in %.3f s (%d checked)" % (res["ops"], res["seconds"], res["checked"]))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
