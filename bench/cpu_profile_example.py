"""The profiling example of the reference's README on CPU ranks: ten all_reduces of a [2,2] and
a [4,4] fp32 tensor under the autograd profiler, then a barrier (README.md:225-252 of
intel/torch-ccl; its published table, README.md:256-283, is the only timing the reference
publishes: first-shape all_reduce 29.8 ms per call including communicator bring-up, [4,4]
all_reduce 19-108 us to enqueue plus 5.7-97 us in the wait range, 326-332 ms in total).

    python bench/cpu_profile_example.py            # spawns 2 ranks, prints rank 0's table and a JSON line
"""
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(rank, world, port):
    import oneccl_bindings_for_pytorch  # noqa: F401

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("ccl", rank=rank, world_size=world)
    x = torch.ones([2, 2])
    y = torch.ones([4, 4])
    t0 = time.perf_counter()
    with torch.autograd.profiler.profile(record_shapes=True) as prof:
        for _ in range(10):
            dist.all_reduce(x)
            dist.all_reduce(y)
    dist.barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    if rank == 0:
        avg = prof.key_averages(group_by_input_shape=True)
        print(avg.table(sort_by="self_cpu_time_total", row_limit=12))
        rows = {}
        for e in avg:
            if e.key.startswith("oneccl_bindings_for_pytorch::"):
                rows["%s %s" % (e.key.split("::", 1)[1], e.input_shapes[:1])] = round(e.cpu_time_total / max(1, e.count), 1)
        print(json.dumps({"bench": "cpu_profile_example", "world": world, "avg_us_per_call": rows, "wall_ms_20_allreduces_and_barrier": round(wall_ms, 2),
                          "reference_published": {"first_shape_allreduce_ms": 29.79, "allreduce_4x4_enqueue_us": [19.0, 108.2],
                                                  "wait_4x4_us": [97.4, 5.7], "self_cpu_total_ms": [325.9, 331.7]}}))
    dist.destroy_process_group()


if __name__ == "__main__":
    mp.spawn(run, args=(2, 29631), nprocs=2)
