"""Headline benchmark: tensor-parallel decode of a Llama-architecture 7B model over the `ccl`
backend (32 layers, hidden 4096, 32 heads of 128, SwiGLU FFN 11008, vocab 32000, bf16 random
N(0, 0.02) weights), batch 16, 1024-token prompt of uniform random ids, TP = number of GPUs.

    python bench.py --gpus N --steps K --warmup W           (N > 1: launched by torchrun)

A "step" generates one token for each of the 16 sequences (one CUDA-graph replay of the whole
decode step: tcgen05 GEMMs, fused RoPE/KV-append/attention, one-shot all_reduce fused with
residual-add + RMSNorm). Rank 0 prints ONE JSON line; `value` is tokens/s of the whole job.
Timing: CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks.
Each step streams the rank's whole weight shard (13.5 GB / N) and KV cache from HBM, far more
than the 126 MB L2, so no L2 flush is needed between steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "tp_decode_tokens_per_s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ccl", choices=["ccl", "reference"])
    ap.add_argument("--collective", default="ccl", choices=["ccl", "nccl"],
                    help="nccl: same model and kernels, all_reduce through torch's NCCL backend + a separate add/norm kernel (comparison arm)")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=32, help="testing only; the headline config has 32")
    ap.add_argument("--no-graph", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = f"/tmp/ccl_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=max(power))
        return out


def reference_arm(args):
    # The reference is a binding over Intel oneCCL for Intel GPUs. Its install was attempted with
    # `pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --target baseline/_ref`
    # and fails in cmake: third_party/oneCCL is an empty submodule ("does not contain a
    # CMakeLists.txt", "Failed to find oneCCL target"), and its device path needs SYCL/Level-Zero.
    print(json.dumps({"impl": "reference", "unavailable":
                      "intel/torch-ccl cannot be built here: third_party/oneCCL is an empty submodule (cmake: 'Failed to find oneCCL target') "
                      "and its GPU path needs SYCL + Level-Zero on Intel GPUs"}))
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus > 1 and "RANK" not in os.environ:
        # convenience: re-launch under torchrun on this node
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    import oneccl_bindings_for_pytorch  # noqa: F401  (registers backend "ccl")
    import torch_ccl_b200._C as C
    from torch_ccl_b200.models.llama import LlamaConfig, TPLlamaDecoder

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("ccl", rank=rank, world_size=world)

    cfg = LlamaConfig.llama7b()
    cfg.n_layers = args.layers
    B, S, K, W = args.batch, args.prompt, args.steps, args.warmup
    max_seq = S + W + 2 * K + 16
    max_seq = (max_seq + 255) // 256 * 256
    model = TPLlamaDecoder(cfg, max_batch=B, max_seq=max_seq, seed=0, collective=args.collective)

    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab, (B, S), generator=g)
    t0 = time.time()
    model.prefill(prompt)
    prefill_s = time.time() - t0
    if not args.no_graph:
        model.capture(B)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def run_steps(n):
        for _ in range(n):
            model.decode_step(B)

    model.decode_step(B)
    for _ in range(W):
        run_steps(1)

    def timed(fn):
        barrier()
        sampler = ClockSampler(local_rank) if rank == 0 else None
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(dev)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        clocks = sampler.stop() if sampler else None
        return float(ms.item()), clocks

    # ---- device-timed region: K decode steps --------------------------------------------------
    C.launch_count_reset()
    # a profiler started with "--profile-from-start off" captures exactly the timed steps
    profile_range = os.environ.get("CCL_BENCH_PROFILE_RANGE") == "1"
    if profile_range:
        torch.cuda.cudart().cudaProfilerStart()
    ms, clocks = timed(lambda: run_steps(K))
    if profile_range:
        torch.cuda.cudart().cudaProfilerStop()
    tokens_per_s = B * K / (ms * 1e-3)

    # ---- end to end through the public API: ids from pinned host memory, result read back ------
    pin_in = torch.zeros(B, dtype=torch.int64).pin_memory()
    pin_out = torch.zeros(B, dtype=torch.int64).pin_memory()
    pin_in.copy_(model.next_tokens[:B].cpu())

    def e2e_loop():
        for _ in range(K):
            model.decode_step_host(pin_in, pin_out)
            pin_in.copy_(pin_out)

    ms_e2e, clocks_e2e = timed(e2e_loop)
    e2e_tokens_per_s = B * K / (ms_e2e * 1e-3)

    if rank == 0:
        out = {
            "metric": METRIC, "value": round(tokens_per_s, 2), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "impl": "ccl" if args.collective == "ccl" else "ccl kernels + nccl all_reduce",
            "config": {"model": "llama-7b-arch (32L, h4096, 32x128 heads, ffn 11008, vocab 32000)" if args.layers == 32 else f"llama-7b-arch truncated to {args.layers} layers (NOT the headline config)",
                       "global_batch": B, "seq_len": S, "new_tokens_timed": K, "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2: every step streams the whole weight shard and KV cache from HBM",
                       "cuda_graph": not args.no_graph, "prefill_s": round(prefill_s, 2)},
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"]},
            "e2e": {"value": round(e2e_tokens_per_s, 2), "unit": "tokens/s", "h2d_bytes_per_step": B * 8,
                    "d2h_bytes_per_step": B * 8, "ms_per_step": round(ms_e2e / K, 4),
                    "clocks": {"sm_mhz": clocks_e2e["sm_mhz"], "reasons": clocks_e2e["reasons"]}},
            "gpu_launches": model.kernels_per_step * K,
            "kernels_per_step": model.kernels_per_step,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
