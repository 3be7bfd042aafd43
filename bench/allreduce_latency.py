"""Kernel-level all_reduce latency of the `ccl` communicator: the collective is enqueued on the
current stream through the fused-op entry (no c10d Work, no event fork/join), so the number is
launch + kernel time. With TORCH_CCL_SYNC_ONLY=1 / TORCH_CCL_WORK_ONLY=1 in the environment the
same kernels run only their flag protocol / only their data movement (the counterpart of the
reference's Synconly / Workonly kernel variants, src/gpu/allreduce_small.h:443-982), which splits
the latency into synchronisation and data time.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/allreduce_latency.py
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oneccl_bindings_for_pytorch  # noqa: E402,F401
from torch_ccl_b200 import get_backend  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("ccl", rank=rank, world_size=world)
    be = get_backend(None, "cuda")
    mode = "sync_only" if os.environ.get("TORCH_CCL_SYNC_ONLY") == "1" else ("work_only" if os.environ.get("TORCH_CCL_WORK_ONLY") == "1" else "full")
    sizes = [8 << 10, 32 << 10, 128 << 10, 512 << 10, 1 << 20, 2 << 20, 4 << 20, 8 << 20, 32 << 20, 128 << 20]
    probe = torch.ones(8, device=dev)
    dist.all_reduce(probe)
    nvls = bool(be.cuda_comm_config(probe)["nvls_available"])  # CCL_NVLS=1: sizes >= 4 MB go through the switch
    for dtype in (torch.bfloat16,):
        for size in sizes:
            t = torch.ones(size // dtype.itemsize, device=dev, dtype=dtype)
            iters = 50 if size <= (8 << 20) else 10
            g = torch.cuda.CUDAGraph()
            be.fused_allreduce(t, 1.0)
            torch.cuda.synchronize()
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                be.fused_allreduce(t, 1.0)
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s):
                for _ in range(iters):
                    be.fused_allreduce(t, 1.0)
            dist.barrier()
            torch.cuda.synchronize()
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev, dtype=torch.float64)
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
            if rank == 0:
                print(json.dumps({"mode": mode, "world": world, "dtype": str(dtype).split(".")[-1], "bytes": size, "us": round(float(us), 2),
                                  "busbw_GBps": round(size * 2 * (world - 1) / world / float(us) / 1e3, 1), "nvls": nvls}), flush=True)
            del g
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
