"""Fused tensor-parallel GEMM + collective ops against cuBLAS + NCCL on the same GPUs.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/fused_gemm_bench.py

gemm_rs:  row-parallel linear (K sharded) + reduce_scatter over rows    [Llama-7B down/o projections]
ag_gemm:  all_gather over rows + column-parallel linear (N sharded)     [Llama-7B gate/up/qkv projections]
Baseline: torch.matmul (cuBLAS) + dist.reduce_scatter_tensor / all_gather_into_tensor on an NCCL group.
Device-timed (CUDA events), max over ranks. Roofline per op: the slower of FLOPs / measured bf16 peak
and NVLink bytes / 770 GB/s (measured peer copy); reported as `roofline_frac` = roofline time / achieved.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oneccl_bindings_for_pytorch  # noqa: E402,F401
from torch_ccl_b200 import ops  # noqa: E402


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def timeit(fn, group, dev, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) * 1e-3


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("ccl", rank=rank, world_size=world)
    nccl = dist.new_group(backend="nccl")
    tf_peak, src = peaks()
    link = 770e9
    M = 8192  # tokens
    rows = []
    # (name, N, K_full) of the row-parallel (gemm_rs) and column-parallel (ag_gemm) projections
    for name, N, K in [("down 11008->4096", 4096, 11008), ("o 4096->4096", 4096, 4096)]:
        Kl = K // world // 8 * 8
        a = torch.randn(M, Kl, device=dev, dtype=torch.bfloat16)
        b = torch.randn(N, Kl, device=dev, dtype=torch.bfloat16) * 0.02
        out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
        full = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        t_f = timeit(lambda: ops.gemm_reduce_scatter(a, b, out=out), None, dev)

        def base():
            torch.matmul(a, b.t(), out=full)
            dist.reduce_scatter_tensor(out, full, group=nccl)

        t_b = timeit(base, nccl, dev)
        flops = 2.0 * M * N * Kl
        roof = max(flops / (tf_peak * 1e12), (M * N * 2) * (world - 1) / world / link)
        rows.append({"op": "gemm_rs", "shape": name, "M": M, "N": N, "K_local": Kl, "world": world,
                     "fused_us": round(t_f * 1e6, 1), "cublas_nccl_us": round(t_b * 1e6, 1),
                     "speedup": round(t_b / t_f, 3), "tflops": round(flops / t_f / 1e12, 1),
                     f"roofline_frac_{src}": round(roof / t_f, 3)})
    for name, N, K in [("gate/up 4096->22016", 22016, 4096), ("qkv 4096->12288", 12288, 4096)]:
        Nl = N // world // 16 * 16
        a = torch.randn(M // world, K, device=dev, dtype=torch.bfloat16)
        b = torch.randn(Nl, K, device=dev, dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, Nl, device=dev, dtype=torch.bfloat16)
        gathered = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        t_f = timeit(lambda: ops.all_gather_gemm(a, b, out=out), None, dev)

        def base():
            dist.all_gather_into_tensor(gathered, a, group=nccl)
            torch.matmul(gathered, b.t(), out=out)

        t_b = timeit(base, nccl, dev)
        flops = 2.0 * M * Nl * K
        roof = max(flops / (tf_peak * 1e12), (M * K * 2) * (world - 1) / world / link)
        rows.append({"op": "ag_gemm", "shape": name, "M": M, "N_local": Nl, "K": K, "world": world,
                     "fused_us": round(t_f * 1e6, 1), "cublas_nccl_us": round(t_b * 1e6, 1),
                     "speedup": round(t_b / t_f, 3), "tflops": round(flops / t_f / 1e12, 1),
                     f"roofline_frac_{src}": round(roof / t_f, 3)})
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
