"""Three DistributedDataParallel iterations of a tiny model on the `ccl` backend, under the
PyTorch profiler, to show where the backend's ranges appear in a profile.

    python demo/demo.py                      # 2 CPU ranks, spawned here
    python demo/demo.py --device cuda        # one rank per visible GPU (needs >= 2)
    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 demo/demo.py [--device cuda]

Rows named `oneccl_bindings_for_pytorch::allreduce` are the backend entry (with input shapes);
`oneccl_bindings_for_pytorch::cpu::allreduce` / `...::cuda::allreduce` are the device-side part.
The names are those of intel/torch-ccl (demo/demo.py and README.md:236-280 there), so profiler
scripts written against it keep working.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oneccl_bindings_for_pytorch  # noqa: E402,F401  (registers the "ccl" backend)


class Model(nn.Module):
    def __init__(self):
        super().__init__()
        self.linear = nn.Linear(4, 5)

    def forward(self, x):
        return self.linear(x)


def run(rank, world, device, spawned):
    if spawned:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=os.environ.get("MASTER_PORT", "29611"))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("ccl", rank=rank, world_size=world)
    dev = torch.device(device, torch.cuda.current_device()) if device == "cuda" else torch.device("cpu")
    model = Model().to(dev)
    ddp = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index] if device == "cuda" else None)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.001)
    loss_fn = nn.MSELoss()
    acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if device == "cuda" else [])
    with torch.profiler.profile(activities=acts, record_shapes=True) as prof:
        for _ in range(3):
            x = torch.randn(2, 4, device=dev)
            y = torch.randn(2, 5, device=dev)
            loss = loss_fn(ddp(x), y)
            opt.zero_grad()
            loss.backward()
            opt.step()
        if device == "cuda":
            torch.cuda.synchronize()
    if rank == 0:
        rows = [e for e in prof.key_averages() if "oneccl_bindings_for_pytorch" in e.key]
        print("%-60s %8s %12s" % ("range", "calls", "cpu total us"))
        for e in sorted(rows, key=lambda e: e.key):
            print("%-60s %8d %12.1f" % (e.key, e.count, e.cpu_time_total))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    a = ap.parse_args()
    if "RANK" in os.environ:
        run(0, 0, a.device, False)
    else:
        world = torch.cuda.device_count() if a.device == "cuda" else 2
        mp.spawn(run, args=(world, a.device, True), nprocs=world)


if __name__ == "__main__":
    main()
