"""Headline benchmark: tensor-parallel decode of a Llama-architecture 7B model over the `ccl`
backend (32 layers, hidden 4096, 32 heads of 128, SwiGLU FFN 11008, vocab 32000, bf16 random
N(0, 0.02) weights), batch 16, 1024-token prompt of uniform random ids, TP = number of GPUs.

    python bench.py --gpus N --steps K --warmup W           (N > 1: launched by torchrun)

A "step" generates one token for each of the 16 sequences (one CUDA-graph replay of the whole
decode step: tcgen05 GEMMs, fused RoPE/KV-append/attention, and each row-parallel projection
fused with its all_reduce + residual-add + RMSNorm in one kernel). Rank 0 prints ONE JSON line;
`value` is tokens/s of the whole job.
Timing: a timed region is K steps between CUDA events on the launching stream, with a barrier +
synchronize on both sides and the max taken over ranks; the region is repeated `--repeats` times
from the same starting context and the MEDIAN is reported (`spread` gives min / max), so that the
clock record holds more than a couple of samples and one slow replay does not move the number.
Each step streams the rank's whole weight shard (13.5 GB / N) and KV cache from HBM, far more
than the 126 MB L2, so no L2 flush is needed between steps.
After the repo's arm the same step is measured in plain PyTorch on the stock stack
(bench/torch_decode_baseline.py: cuBLAS matmul, SDPA, rms_norm, NCCL all_reduce, CUDA graph);
`vs_baseline` is tokens/s of this repo divided by tokens/s of that arm on the same GPUs.
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
    ap.add_argument("--repeats", type=int, default=7, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--unfused", action="store_true", help="separate GEMM / all_reduce+norm / sampling kernels (A/B of the fused decode kernels)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the plain-PyTorch + NCCL comparison arm")
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
    B, S, K, W, R = args.batch, args.prompt, args.steps, args.warmup, max(1, args.repeats)
    max_seq = (S + max(K, W) + 16 + 255) // 256 * 256

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def measure(run_region, reset):
        """R timed regions; returns (list of ms per region, max over ranks each; clock record)."""
        sampler = ClockSampler(local_rank) if rank == 0 else None
        if sampler:
            sampler.start()
        out = []
        for _ in range(R):
            reset()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run_region()
            e1.record()
            torch.cuda.synchronize(dev)
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            out.append(float(ms.item()))
        clocks = sampler.stop() if sampler else None
        return out, clocks

    def summarize(ms_list):
        med = statistics.median(ms_list)
        return {"tokens_per_s": B * K / (med * 1e-3), "ms_per_step": med / K, "min_ms_per_step": min(ms_list) / K,
                "max_ms_per_step": max(ms_list) / K, "regions": [round(m / K, 4) for m in ms_list]}

    # ---- this repository's arm ----------------------------------------------------------------------
    model = TPLlamaDecoder(cfg, max_batch=B, max_seq=max_seq, seed=0, collective=args.collective, fused=not args.unfused)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab, (B, S), generator=g)
    barrier()
    t0 = time.time()
    model.prefill(prompt)
    barrier()
    prefill_s = time.time() - t0
    if not args.no_graph:
        model.capture(B)
    model.decode_step(B)
    for _ in range(W):
        model.decode_step(B)

    def reset_model():
        model.positions[:B] = S  # every region decodes the same K positions after the prompt

    C.launch_count_reset()
    # a profiler started with "--profile-from-start off" captures exactly the timed steps
    profile_range = os.environ.get("CCL_BENCH_PROFILE_RANGE") == "1"
    if profile_range:
        torch.cuda.cudart().cudaProfilerStart()

    def region():
        for _ in range(K):
            model.decode_step(B)

    ms_list, clocks = measure(region, reset_model)
    if profile_range:
        torch.cuda.cudart().cudaProfilerStop()
    dev_res = summarize(ms_list)

    # ---- end to end through the public API: ids from pinned host memory, result read back ------
    pin_in = torch.zeros(B, dtype=torch.int64).pin_memory()
    pin_out = torch.zeros(B, dtype=torch.int64).pin_memory()
    pin_in.copy_(model.next_tokens[:B].cpu())

    def e2e_region():
        for _ in range(K):
            model.decode_step_host(pin_in, pin_out)
            pin_in.copy_(pin_out)

    ms_e2e, clocks_e2e = measure(e2e_region, reset_model)
    e2e_res = summarize(ms_e2e)

    if os.environ.get("CCL_BENCH_KERNEL_TABLE") and rank == 0:
        # diagnostic only (never a bench value): per-kernel device time of a few graph replays, as seen by torch's profiler
        from torch.profiler import ProfilerActivity, profile

        reset_model()
        torch.cuda.synchronize(dev)
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                model.decode_step(B)
            torch.cuda.synchronize(dev)
        with open(os.environ["CCL_BENCH_KERNEL_TABLE"], "w") as f:
            f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=30, max_name_column_width=90))
    elif os.environ.get("CCL_BENCH_KERNEL_TABLE"):
        reset_model()
        for _ in range(3):
            model.decode_step(B)
        torch.cuda.synchronize(dev)
    kernels_per_step = model.kernels_per_step
    fused = model.fused
    del model
    torch.cuda.empty_cache()

    # ---- comparison arm: plain PyTorch (cuBLAS, SDPA, rms_norm) + NCCL, same shapes, CUDA graph --------
    base = None
    if not args.no_baseline:
        import importlib.util

        spec = importlib.util.spec_from_file_location("torch_decode_baseline", os.path.join(ROOT, "bench", "torch_decode_baseline.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        TorchTPDecoder = mod.TorchTPDecoder

        nccl = dist.new_group(backend="nccl") if world > 1 else None
        kv_len = (S + max(K, W) + 8 + 63) // 64 * 64
        tm = TorchTPDecoder(cfg, B, S, kv_len, group=nccl, device=dev, seed=1)
        if not args.no_graph:
            tm.capture()
        for _ in range(W + 1):
            tm.decode_step()

        def reset_tm():
            tm.positions.fill_(S)

        def tm_region():
            for _ in range(K):
                tm.decode_step()

        b_ms, b_clocks = measure(tm_region, reset_tm)
        pin_in.copy_(tm.next_tokens.cpu())

        def tm_e2e():
            for _ in range(K):
                tm.decode_step_host(pin_in, pin_out)
                pin_in.copy_(pin_out)

        b_e2e_ms, _ = measure(tm_e2e, reset_tm)
        bd, be = summarize(b_ms), summarize(b_e2e_ms)
        base = {"impl": "plain PyTorch: torch.matmul (cuBLAS), scaled_dot_product_attention, rms_norm, eager RoPE / KV append, "
                        "NCCL all_reduce + all_gather, one CUDA graph per step; none of this repository's kernels",
                "tokens_per_s": round(bd["tokens_per_s"], 2), "ms_per_step": round(bd["ms_per_step"], 4),
                "e2e_tokens_per_s": round(be["tokens_per_s"], 2),
                "ratio": round(dev_res["tokens_per_s"] / bd["tokens_per_s"], 4),
                "e2e_ratio": round(e2e_res["tokens_per_s"] / be["tokens_per_s"], 4),
                "clocks": {"sm_mhz": b_clocks["sm_mhz"], "reasons": b_clocks["reasons"]} if b_clocks else None}
        del tm

    if rank == 0:
        out = {
            "metric": METRIC, "value": round(dev_res["tokens_per_s"], 2), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": round(dev_res["ms_per_step"], 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": base["ratio"] if base else None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "impl": ("ccl" if fused else "ccl, unfused decode kernels") if args.collective == "ccl" else "ccl kernels + nccl all_reduce",
            "repeats": R, "spread": {"min_ms_per_step": round(dev_res["min_ms_per_step"], 4), "max_ms_per_step": round(dev_res["max_ms_per_step"], 4),
                                     "ms_per_step_of_each_region": dev_res["regions"]},
            "config": {"model": "llama-7b-arch (32L, h4096, 32x128 heads, ffn 11008, vocab 32000)" if args.layers == 32 else f"llama-7b-arch truncated to {args.layers} layers (NOT the headline config)",
                       "global_batch": B, "seq_len": S, "new_tokens_timed": K, "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2: every step streams the whole weight shard and KV cache from HBM",
                       "timing": f"median of {R} regions of {K} steps, each from context {S}",
                       "cuda_graph": not args.no_graph, "prefill_s": round(prefill_s, 2)},
            "prefill_tokens_per_s": round(B * S / prefill_s, 1),
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"]},
            "e2e": {"value": round(e2e_res["tokens_per_s"], 2), "unit": "tokens/s", "h2d_bytes_per_step": B * 8,
                    "d2h_bytes_per_step": B * 8, "ms_per_step": round(e2e_res["ms_per_step"], 4),
                    "ms_per_step_of_each_region": e2e_res["regions"],
                    "clocks": {"sm_mhz": clocks_e2e["sm_mhz"], "reasons": clocks_e2e["reasons"]}},
            "gpu_launches": kernels_per_step * K,
            "kernels_per_step": kernels_per_step,
            "baseline": base,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
