"""Device-timed throughput of the tcgen05 bf16 GEMM on decode (swap-AB) and training shapes.

Each timed call works on operands cycled through a pool larger than the 126 MB L2, so weight
bytes really come from HBM. Reports achieved GB/s (memory-bound decode shapes) or TFLOP/s and the
fraction of the measured peaks in MEASURED_PEAKS.json (fallback 6650 GB/s, 1590 TFLOP/s).
"""
import argparse
import json
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch_ccl_b200._C as C  # noqa: E402
from torch_ccl_b200.ops import pack_weight  # noqa: E402


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters, warmup=5):
    for _ in range(warmup):
        fn(0)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(iters):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--torch", action="store_true", help="also time torch.matmul (cuBLAS)")
    args = ap.parse_args()
    hbm, tf, src = peaks()
    rows = []
    # (label, n_out, K, batch, dual, splitk)
    decode = [
        ("qkv tp1", 12288, 4096, 16, 0, 0), ("o tp1", 4096, 4096, 16, 0, 0),
        ("gateup tp1", 11008, 4096, 16, 1, 0), ("down tp1", 4096, 11008, 16, 0, 0),
        ("lm_head tp1", 32000, 4096, 16, 0, 0),
        ("qkv tp8", 1536, 4096, 16, 0, 0), ("o tp8", 4096, 512, 16, 0, 0),
        ("gateup tp8", 1376, 4096, 16, 1, 0), ("down tp8", 4096, 1376, 16, 0, 0),
    ]
    for label, n_out, K, batch, dual, splitk in decode:
        wrows = n_out * (2 if dual else 1)
        nbuf = max(2, int(300e6 // (wrows * K * 2)) + 1)
        ws = [torch.randn(wrows, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(nbuf)]
        x = torch.randn(batch, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(batch, n_out, device="cuda", dtype=torch.bfloat16)
        t = timeit(lambda i: C.gemm_bf16_tn(ws[i % nbuf], x, out, True, n_out if dual else 0, splitk, 16), args.iters)
        gbs = wrows * K * 2 / t / 1e9
        row = {"shape": label, "us": round(t * 1e6, 2), "GBps": round(gbs, 1), f"frac_hbm_{src}": round(gbs / hbm, 3)}
        # the same product with the weights pre-packed as contiguous 128x64 tiles
        pad = (n_out + 127) // 128 * 128
        if dual:
            pk = [torch.cat([pack_weight(w[:n_out]), pack_weight(w[n_out:])]) for w in ws]
        else:
            pk = [pack_weight(w) for w in ws]
        t2 = timeit(lambda i: C.gemm_bf16_tn(pk[i % nbuf], x, out, True, pad if dual else 0, splitk, 16, n_out), args.iters)
        row["tiled_us"] = round(t2 * 1e6, 2)
        row[f"tiled_frac_hbm_{src}"] = round(wrows * K * 2 / t2 / 1e9 / hbm, 3)
        del pk
        if args.torch and not dual:
            tt = timeit(lambda i: torch.matmul(x, ws[i % nbuf].t(), out=out), args.iters)
            row["torch_us"] = round(tt * 1e6, 2)
        rows.append(row)
        del ws
    for M, N, K in [(8192, 8192, 8192), (16384, 4096, 4096), (2048, 11008, 4096), (2048, 4096, 11008)]:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t = timeit(lambda i: C.gemm_bf16_tn(a, b, out, False, 0, 1, 0), max(5, args.iters // 5))
        tfs = 2.0 * M * N * K / t / 1e12
        row = {"shape": f"{M}x{N}x{K}", "us": round(t * 1e6, 1), "TFLOPs": round(tfs, 1), f"frac_bf16_{src}": round(tfs / tf, 3)}
        if args.torch:
            tt = timeit(lambda i: torch.matmul(a, b.t(), out=out), max(5, args.iters // 5))
            row["torch_TFLOPs"] = round(2.0 * M * N * K / tt / 1e12, 1)
        rows.append(row)
    for r in rows:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
